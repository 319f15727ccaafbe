// Library-wide pieces of the C ABI: last-error text, device status word, launch counter, tensor-map encoder.
#include "es_api_internal.h"
#include "es_ptx.cuh"

#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

namespace es {

static thread_local char g_error[512] = "";
static std::atomic<long long> g_launches{0};

// Written by a kernel whose bounded wait ran out (the code says which wait). One word per device, in that device's
// copy of this module.
__device__ int g_status_word = 0;

int set_error(int code, const char* msg) {
    std::snprintf(g_error, sizeof(g_error), "%s", msg ? msg : "");
    return code;
}

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int* device_status_ptr() {
    static int* ptrs[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!ptrs[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
        ptrs[dev] = static_cast<int*>(p);
    }
    return ptrs[dev];
}

// cudaFuncAttributeMaxDynamicSharedMemorySize is a property of (kernel, device): a process that uses several GPUs has
// to opt in on each of them. The pairs already done are remembered, so a launch costs one short list walk.
int opt_in_shared_memory(const void* kernel, int bytes) {
    struct Done { int dev; const void* kernel; int bytes; };
    static std::mutex mu;
    static std::vector<Done> done;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return set_error(-2, cudaGetErrorString(e));
    std::lock_guard<std::mutex> lock(mu);
    for (const Done& d : done)
        if (d.dev == dev && d.kernel == kernel && d.bytes >= bytes) return 0;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return set_error(-2, cudaGetErrorString(e));
    done.push_back({dev, kernel, bytes});
    return 0;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

int encode_tensor_map(CUtensorMap* m, CUtensorMapDataType dt, uint32_t rank, void* base, const cuuint64_t* dims,
                      const cuuint64_t* strides_bytes, const cuuint32_t* box, const cuuint32_t* elem_strides,
                      CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return set_error(-3, "cuTensorMapEncodeTiled is not available from this driver");
    CUresult r = fn(m, dt, rank, base, dims, strides_bytes, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char buf[128];
        std::snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return set_error(-3, buf);
    }
    return 0;
}

// A wait that nothing ends: one warp waits on a barrier nobody arrives on, with a short limit. It takes the same path
// as a wait of the attention kernels that runs out: the code goes to the status word, the kernel returns.
__global__ void selftest_wait_kernel(int* status, unsigned long long limit_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncwarp();
    mbar_wait(smem_u32(&bar), 0, &abort_flag, status, 777, 0, limit_ns);
}

}  // namespace es

extern "C" int es_selftest_wait_timeout(int32_t limit_us, void* stream) {
    if (limit_us < 1 || limit_us > 100000) return es::set_error(-1, "es_selftest_wait_timeout: limit must be 1 .. 100000 us");
    int* st = es::device_status_ptr();
    if (!st) return es::set_error(-2, "es_selftest_wait_timeout: the device status word is not available");
    es::selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(st, (unsigned long long)limit_us * 1000ull);
    ES_CHECK_LAUNCH("selftest_wait");
    return 0;
}

extern "C" const char* es_last_error(void) { return es::g_error; }

extern "C" int es_abi_version(void) { return 1; }

extern "C" long long es_launch_count(void) { return es::g_launches.load(std::memory_order_relaxed); }

// Reads the status word of the current device and clears it. Synchronises the device.
extern "C" int es_device_status(int32_t* status_out) {
    int* p = es::device_status_ptr();
    if (!p || !status_out) return es::set_error(-1, "es_device_status: no device or null pointer");
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return es::set_error(-2, cudaGetErrorString(e));
    int v = 0;
    e = cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return es::set_error(-2, cudaGetErrorString(e));
    *status_out = v;
    if (v != 0) {
        int zero = 0;
        cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice);
    }
    return 0;
}
