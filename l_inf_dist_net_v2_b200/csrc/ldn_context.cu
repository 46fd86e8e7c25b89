// Host-side context: cached device properties, per-(device, stream) scratch arenas, TMA descriptor
// construction through the driver entry point (no link-time dependency on libcuda).
#include <mutex>
#include <vector>

#include "ldn_common.cuh"

namespace ldn {

namespace {
std::mutex g_mutex;
DeviceCtx g_ctx[64];
bool g_ctx_ready[64] = {};

struct ArenaEntry {
    int device;
    cudaStream_t stream;
    Arena arena;
};
std::vector<ArenaEntry*> g_arenas;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
}  // namespace

int get_device_ctx(const DeviceCtx** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return kNoDevice;
    if (dev < 0 || dev >= 64) return kNoDevice;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_ctx_ready[dev]) {
        DeviceCtx c;
        c.device = dev;
        if (cudaDeviceGetAttribute(&c.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return kNoDevice;
        if (cudaDeviceGetAttribute(&c.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess)
            return kNoDevice;
        g_ctx[dev] = c;
        g_ctx_ready[dev] = true;
    }
    *out = &g_ctx[dev];
    return kOk;
}

// Finds (or creates, with its status word) the arena of (current device, stream).  Never touches the scratch block.
int find_arena(cudaStream_t stream, Arena** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return kNoDevice;
    std::lock_guard<std::mutex> lock(g_mutex);
    ArenaEntry* ent = nullptr;
    for (ArenaEntry* a : g_arenas)
        if (a->device == dev && a->stream == stream) ent = a;
    if (!ent) {
        ent = new ArenaEntry();
        ent->device = dev;
        ent->stream = stream;
        ent->arena = Arena{nullptr, 0, nullptr, nullptr, new std::mutex(), false, new std::vector<void*>()};
        auto drop = [&]() {
            delete static_cast<std::mutex*>(ent->arena.call_mutex);
            delete static_cast<std::vector<void*>*>(ent->arena.retired);
            delete ent;
        };
        if (cudaMalloc(&ent->arena.status, 256) != cudaSuccess) {
            drop();
            return kWorkspace;
        }
        cudaMemset(ent->arena.status, 0, 256);
        if (cudaMallocHost(&ent->arena.status_host, sizeof(int)) != cudaSuccess) {
            cudaFree(ent->arena.status);
            drop();
            return kWorkspace;
        }
        *ent->arena.status_host = 0;
        g_arenas.push_back(ent);
    }
    *out = &ent->arena;
    return kOk;
}

// Makes the arena's block at least `bytes` large.  The caller holds the arena's call mutex, so no other host thread
// is enqueueing kernels that use the block.  While the stream is being captured nothing may be allocated or waited
// for, so a growth is refused then; and once a capture has used the arena, earlier blocks are kept (a captured
// graph replays with the addresses it was recorded with) until ldn_release_scratch.
int ensure_arena(Arena* arena, cudaStream_t stream, size_t bytes) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess) {
        cudaGetLastError();
        cs = cudaStreamCaptureStatusNone;
    }
    const bool capturing = cs != cudaStreamCaptureStatusNone;
    if (capturing) arena->graph_used = true;
    if (bytes <= arena->capacity) return kOk;
    if (capturing) return kCaptureGrowth;
    // kernels already queued on the stream may still use the old block
    cudaStreamSynchronize(stream);
    if (arena->base) {
        if (arena->graph_used) static_cast<std::vector<void*>*>(arena->retired)->push_back(arena->base);
        else cudaFree(arena->base);
    }
    arena->base = nullptr;
    const size_t old_cap = arena->capacity;
    arena->capacity = 0;
    size_t want = bytes + bytes / 8;
    // kept blocks add up: grow geometrically then, so that they stay below twice the final size
    if (arena->graph_used && want < old_cap + old_cap / 2) want = old_cap + old_cap / 2;
    want = (want + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    void* p = nullptr;
    if (cudaMalloc(&p, want) != cudaSuccess) {
        cudaGetLastError();
        if (cudaMalloc(&p, bytes) != cudaSuccess) {
            cudaGetLastError();
            return kWorkspace;
        }
        want = bytes;
    }
    arena->base = static_cast<char*>(p);
    arena->capacity = want;
    return kOk;
}

int release_arenas() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return kNoDevice;
    cudaDeviceSynchronize();
    std::lock_guard<std::mutex> lock(g_mutex);
    std::vector<ArenaEntry*> keep;
    for (ArenaEntry* a : g_arenas) {
        if (a->device != dev) {
            keep.push_back(a);
            continue;
        }
        if (a->arena.base) cudaFree(a->arena.base);
        auto* retired = static_cast<std::vector<void*>*>(a->arena.retired);
        for (void* p : *retired) cudaFree(p);
        delete retired;
        cudaFree(a->arena.status);
        cudaFreeHost(a->arena.status_host);
        delete static_cast<std::mutex*>(a->arena.call_mutex);
        delete a;
    }
    g_arenas.swap(keep);
    return kOk;
}

int make_tensor_map(CUtensorMap* map, const float* base, const unsigned long long dims[3],
                    const unsigned long long strides_elems[2], const unsigned box[3], bool swizzle128) {
    if (!g_encode) {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!g_encode) {
            void* fn = nullptr;
            cudaDriverEntryPointQueryResult qres;
            cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
            if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) return kNoDevice;
            g_encode = reinterpret_cast<EncodeTiledFn>(fn);
        }
    }
    cuuint64_t gdim[3] = {dims[0], dims[1], dims[2]};
    cuuint64_t gstr[2] = {strides_elems[0] * 4ull, strides_elems[1] * 4ull};
    cuuint32_t bdim[3] = {box[0], box[1], box[2]};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), gdim, gstr, bdim, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? kOk : kTensorMap;
}

}  // namespace ldn
