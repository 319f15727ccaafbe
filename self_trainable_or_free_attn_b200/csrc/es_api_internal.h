// Host-side helpers shared by the .cu files of the library: error reporting, the device status word that kernels write
// when a bounded wait gives up, the tensor-map encoder (looked up from the driver at run time, so the library does not
// link libcuda), and the launch counter that the benchmark reports.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace es {

// Records `msg` as the last error of this thread and returns `code` (negative).
int set_error(int code, const char* msg);
// Address of this device's status word (0 = fine; otherwise the code of the first wait that gave up).
int* device_status_ptr();
// One more kernel launched by this library (read with es_launch_count).
void count_launch();

// Lets `kernel` use `bytes` of dynamic shared memory on the current device (once per device and kernel). 0 or an error code.
int opt_in_shared_memory(const void* kernel, int bytes);

int encode_tensor_map(CUtensorMap* m, CUtensorMapDataType dt, uint32_t rank, void* base, const cuuint64_t* dims,
                      const cuuint64_t* strides_bytes, const cuuint32_t* box, const cuuint32_t* elem_strides,
                      CUtensorMapSwizzle swizzle);

#define ES_CHECK_LAUNCH(name)                                                     \
    do {                                                                          \
        cudaError_t e__ = cudaGetLastError();                                     \
        if (e__ != cudaSuccess) return es::set_error(-2, cudaGetErrorString(e__)); \
        es::count_launch();                                                       \
    } while (0)

}  // namespace es
