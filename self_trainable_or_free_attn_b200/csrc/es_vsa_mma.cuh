// Warp-level building blocks of the VSA2 kernels: 64 x D token tiles in shared memory (16-byte chunks XOR-swizzled by
// the row, filled with cp.async), ldmatrix fragment loads and m16n8k16 tensor-core MMAs for bf16 and fp16.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace es {
namespace vsa {

constexpr int TB = 64;                 // tokens per block
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

template <typename T> struct Elt;
template <> struct Elt<__nv_bfloat16> {
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    static __device__ __forceinline__ float2 unpack(uint32_t w) {
        return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w));
    }
    static __device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
    static __device__ __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
    static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};
template <> struct Elt<__half> {
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __half2 v = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    static __device__ __forceinline__ float2 unpack(uint32_t w) { return __half22float2(*reinterpret_cast<__half2*>(&w)); }
    static __device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
    static __device__ __forceinline__ __half from_float(float x) { return __float2half_rn(x); }
    static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void cp16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// A tile is 64 rows of D elements (2 D bytes per row); chunk c (16 bytes) of row r sits at chunk c ^ (r & 7).
template <int D> __device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return (uint32_t)(row * D * 2 + ((chunk ^ (row & 7)) << 4));
}
// All 128 threads copy one 64 x D tile (rows of `src` are `ld` elements apart).
template <typename T, int D> __device__ __forceinline__ void load_tile(uint32_t tile, const T* src, size_t ld, int tid) {
    constexpr int CH = D / 8;                         // chunks per row
#pragma unroll
    for (int i = 0; i < TB * CH / 128; ++i) {
        const int idx = i * 128 + tid, row = idx / CH, ch = idx % CH;
        cp16(tile + tile_off<D>(row, ch), src + (size_t)row * ld + ch * 8);
    }
}

// A fragments (16 rows x 16 k) of rows [row0, row0 + 16) for k step ks, from a row-major tile [row][k].
template <int D> __device__ __forceinline__ void load_a(uint32_t tile, int row0, int ks, int lane, uint32_t (&a)[4]) {
    const int row = row0 + (lane & 15), ch = 2 * ks + (lane >> 4);
    ldsm4(tile + tile_off<D>(row, ch), a[0], a[1], a[2], a[3]);
}
// B fragments of the n tiles 2 np and 2 np + 1 (8 columns each) for k step ks, from a tile stored [n][k] (the "K^T" use):
// b[0], b[1] belong to n tile 2 np, b[2], b[3] to 2 np + 1.
template <int D> __device__ __forceinline__ void load_b_nk(uint32_t tile, int np, int ks, int lane, uint32_t (&b)[4]) {
    const int row = np * 16 + ((lane >> 4) << 3) + (lane & 7), ch = 2 * ks + ((lane >> 3) & 1);
    ldsm4(tile + tile_off<D>(row, ch), b[0], b[1], b[2], b[3]);
}
// B fragments of the n tiles 2 dp and 2 dp + 1 for k step kt (16 rows of the tile), from a tile stored [k][n] (the "V" use).
template <int D> __device__ __forceinline__ void load_b_kn(uint32_t tile, int kt, int dp, int lane, uint32_t (&b)[4]) {
    const int row = kt * 16 + (((lane >> 3) & 1) << 3) + (lane & 7), ch = 2 * dp + (lane >> 4);
    ldsm4t(tile + tile_off<D>(row, ch), b[0], b[1], b[2], b[3]);
}

__device__ __forceinline__ float quad_max(float x) {
    x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 1));
    return fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 2));
}
__device__ __forceinline__ float quad_sum(float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    return x + __shfl_xor_sync(0xffffffffu, x, 2);
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace vsa
}  // namespace es
