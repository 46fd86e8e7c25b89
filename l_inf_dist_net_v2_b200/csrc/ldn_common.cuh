// Shared definitions for the sm_100a L_p-distance kernels: tile geometry, kernel parameter blocks,
// mbarrier / TMA primitives (inline PTX, no multicast), and the host-side context.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ldn {

// ---------------------------------------------------------------------------------------------
// Status codes returned by every C-ABI entry point (0 = success).  Values >= 1000 wrap a
// cudaError_t (code - 1000).
// ---------------------------------------------------------------------------------------------
enum Status : int {
    kOk = 0,
    kBadArgument = 1,      // null pointer, non-positive size, CI or CO not divisible by G, p <= 0 ...
    kNoDevice = 2,         // no CUDA device / driver entry point missing
    kWorkspace = 3,        // workspace allocation failed or fixed scratch too small
    kDeviceTimeout = 4,    // a bounded wait inside a kernel gave up (status word set by the device)
    kTensorMap = 5,        // cuTensorMapEncodeTiled rejected a descriptor
    kCaptureGrowth = 6,    // the scratch arena would have to grow while its stream is being captured
    kCudaBase = 1000
};

// ---------------------------------------------------------------------------------------------
// Tile geometry.  One CTA of 256 threads owns a 128 x 128 output tile; every thread owns an
// 8 x 8 register block.  The reduction dimension advances 32 elements per pipeline stage.
// ---------------------------------------------------------------------------------------------
constexpr int kTileM = 128;
constexpr int kTileN = 128;
constexpr int kTileK = 32;
constexpr int kThreads = 256;
constexpr int kRegM = 8;
constexpr int kRegN = 8;
constexpr int kTileElems = kTileM * kTileN;            // outputs per tile
constexpr int kOperandTileBytes = kTileM * kTileK * 4;  // 16 KiB, both operand tile shapes

// Bounded waits: a poll loop gives up after this many failed polls (each followed by a short
// nanosleep once the fast polls are used up), writes kDeviceTimeout into the status word and the
// CTA returns.  2^22 polls * >= 64 ns is far beyond any legitimate TMA latency.
constexpr uint32_t kFastPolls = 1u << 14;
constexpr uint32_t kMaxPolls = 1u << 22;

// One operand as the generic (non-TMA) code sees it: element (row r, inner index c, group g)
// lives at ptr[c + r * stride_row + g * stride_group].
struct Operand {
    const float* ptr;
    long long stride_row;
    long long stride_group;
};

// Output addressing shared by all kernels:
//   offset(m, n, g) = (m / hw_div) * s_b + (m % hw_div) * s_hw + g * s_g + n * s_n
struct OutAddr {
    long long s_b, s_hw, s_g, s_n;
    int hw_div;
};

struct TileParams {
    int M, N, K, G;             // per-group extents of the tile problem
    int tiles_m, tiles_n, kt;   // kt = ceil(K / 32)
    long long total_iters;      // G * tiles_m * tiles_n * kt
    int a_row_coord;            // which TMA coordinate (1 or 2) is the row/k index of A; the other is g
    int b_row_coord;            // same for B
    int b_group_mod;            // > 0: B's group coordinate is (engine group) % b_group_mod; 0: the engine group
    Operand a0, a1, b, pres;    // generic views (rescan of argmax chunks, resident per-output operand)
    OutAddr out;
    float* out_f0;
    float* out_f1;
    int* out_i0;
    int* out_i1;
    float p;                    // the exponent the op was called with
    float q;                    // op specific (p - 1 for backward)
    const float* norm_rows;     // FwdPowNorm with a separable normaliser M[m, n] = max(norm_rows[g][m] + norm_cols[g'][n], 1e-10)
    const float* norm_cols;     //   (row-wise largest magnitudes of the two operands: an upper bound of max |t|); else null
    int* guard;                 // raised by that form when a sum comes out too small for the normaliser to have been adequate
    const float* col_sub;       // optional per-output-channel epilogue of the no-grad p = inf kernels:
    const float* col_add;       //   stored value = (result - col_sub[channel]) + col_add[channel]; either may be null
    const int* gate;            // not null: the kernel returns at once unless (*gate != 0) == (gate_invert == 0)
    int gate_invert;
    int accumulate_out;         // backward kernels: add to the output instead of overwriting it
    float* side_out;            // fused backward: per-row-tile column sums [tile_m][g][k][n] (else null)
    float* partials;            // stream-K scratch: [grid][2][arrays][kTileElems]
    int* status;                // device status word (0 = ok)
    unsigned long long* trace;  // optional per-CTA trace: {sm id, start ns, end ns, iterations}; may be null
};

// ---------------------------------------------------------------------------------------------
// Device primitives
// ---------------------------------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when it gave up.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < kMaxPolls; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i >= kFastPolls) __nanosleep(64);
    }
    return false;
}

// Tiled TMA load of one 3-D box into shared memory (no multicast), completion on an mbarrier.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)),
          "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned sm_id() {
    unsigned s;
    asm volatile("mov.u32 %0, %smid;" : "=r"(s));
    return s;
}

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
#endif  // __CUDACC__

// ---------------------------------------------------------------------------------------------
// Host-side context (ldn_context.cu)
// ---------------------------------------------------------------------------------------------
struct DeviceCtx {
    int device;
    int sm_count;
    int max_smem_optin;
};

// Cached per-device properties for the current device; nullptr + status on failure.
int get_device_ctx(const DeviceCtx** out);

// Per-(device, stream) scratch arena owned by the library.  The block grows on demand (never while the stream is
// being captured) and is 256-byte aligned.  The arena also carries the device status word.
struct Arena {
    char* base;
    size_t capacity;
    int* status;   // device int, zeroed at creation
    int* status_host;  // pinned host mirror used when checking
    void* call_mutex;  // std::mutex*: held for the length of one entry-point call, so that two host threads that
                       // use the same stream cannot interleave launches that share the scratch block
    bool graph_used;   // a call was issued on this arena while its stream was being captured
    void* retired;     // std::vector<void*>*: earlier blocks that captured graphs may still refer to
};
int find_arena(cudaStream_t stream, Arena** out);
int ensure_arena(Arena* arena, cudaStream_t stream, size_t bytes);  // caller holds call_mutex

// Bump allocator over an arena (256-byte granularity).
struct Bump {
    char* base;
    size_t off;
    size_t cap;
    template <class T>
    T* take(size_t count) {
        size_t bytes = (count * sizeof(T) + 255) & ~size_t(255);
        if (off + bytes > cap) return nullptr;
        T* p = reinterpret_cast<T*>(base + off);
        off += bytes;
        return p;
    }
};
inline size_t pad256(size_t bytes) { return (bytes + 255) & ~size_t(255); }

// Tiled 3-D tensor map over fp32 data.  dims/strides are in elements, innermost first; `swizzle128`
// selects the 128-byte swizzle (inner box must then be 32 floats).
int make_tensor_map(CUtensorMap* map, const float* base, const unsigned long long dims[3],
                    const unsigned long long strides_elems[2], const unsigned box[3], bool swizzle128);

// optional CUDA-event pair around the most recent tile-kernel launch (ldn_diag.cu); no-ops unless enabled
void timing_before(cudaStream_t st);
void timing_after(cudaStream_t st);

// host-side launch counter and optional per-CTA trace buffer (ldn_diag.cu)
unsigned long long* trace_buffer();
void count_launches(int n);

inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? kOk : kCudaBase + static_cast<int>(e); }

}  // namespace ldn
