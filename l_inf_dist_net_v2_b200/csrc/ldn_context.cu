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

int get_arena(cudaStream_t stream, size_t bytes, Arena** out) {
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
        ent->arena = Arena{nullptr, 0, nullptr, nullptr, new std::mutex()};
        if (cudaMalloc(&ent->arena.status, 256) != cudaSuccess) {
            delete static_cast<std::mutex*>(ent->arena.call_mutex);
            delete ent;
            return kWorkspace;
        }
        cudaMemset(ent->arena.status, 0, 256);
        if (cudaMallocHost(&ent->arena.status_host, sizeof(int)) != cudaSuccess) {
            cudaFree(ent->arena.status);
            delete static_cast<std::mutex*>(ent->arena.call_mutex);
            delete ent;
            return kWorkspace;
        }
        *ent->arena.status_host = 0;
        g_arenas.push_back(ent);
    }
    if (bytes > ent->arena.capacity) {
        // kernels already queued on the stream may still use the old block
        cudaStreamSynchronize(stream);
        if (ent->arena.base) cudaFree(ent->arena.base);
        ent->arena.base = nullptr;
        ent->arena.capacity = 0;
        size_t want = bytes + bytes / 8;
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
        ent->arena.base = static_cast<char*>(p);
        ent->arena.capacity = want;
    }
    *out = &ent->arena;
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
