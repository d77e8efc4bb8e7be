// Shared device helpers for the sm_100a kernels: status codes, PTX wrappers (mma.sync, ldmatrix,
// cp.async, vector reductions) and fp16 packing.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nerf_b200.h"

#define NB_CHECK_LAUNCH()                                   \
    do {                                                    \
        cudaError_t e_ = cudaGetLastError();                \
        if (e_ != cudaSuccess) return nb_set_cuda_error(e_); \
    } while (0)

#define NB_CUDA(call)                                        \
    do {                                                     \
        cudaError_t e_ = (call);                             \
        if (e_ != cudaSuccess) return nb_set_cuda_error(e_); \
    } while (0)

int nb_set_cuda_error(cudaError_t e);
int nb_set_error(int code, const char* msg);
int nb_num_sms();

namespace nb {

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float2 unpack_half2(uint32_t v) {
    return __half22float2(*reinterpret_cast<__half2*>(&v));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t& r0, uint32_t& r1, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n"
                 : "=r"(r0), "=r"(r1)
                 : "r"(smem_u32(p)));
}

// 16-byte asynchronous global->shared copy; src_bytes = 0 zero-fills the destination.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    int src = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

// Two-wide fp32 reduction to global memory (one L2 atomic for a feature pair).
__device__ __forceinline__ void red_add_v2(float* addr, float a, float b) {
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};\n" ::"l"(addr), "f"(a), "f"(b) : "memory");
}
// Four-wide: two adjacent feature pairs (16-byte aligned address).
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
// fp16 pair reductions (the half-precision gradient table): one entry, or two entries in an aligned 8-byte slot pair.
__device__ __forceinline__ void red_add_h2(uint32_t* addr, uint32_t v) {
    asm volatile("red.global.add.noftz.f16x2 [%0], %1;\n" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_h2x2(uint32_t* addr, uint32_t lo, uint32_t hi) {
    asm volatile("red.global.add.noftz.v2.f16x2 [%0], {%1, %2};\n" ::"l"(addr), "r"(lo), "r"(hi) : "memory");
}
__device__ __forceinline__ void red_add(float* addr, float a) {
    asm volatile("red.global.add.f32 [%0], %1;\n" ::"l"(addr), "f"(a) : "memory");
}

__device__ __forceinline__ void st_cs_v4(void* addr, uint4 v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"l"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ float4 ld_nc_f4(const float* p) {
    float4 v;
    asm volatile("ld.global.nc.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ float contract_axis(float v) {
    return fabsf(v) <= 1.0f ? v : (2.0f - 1.0f / fabsf(v)) * copysignf(1.0f, v);
}

// World position -> the unit cube the hash grid is defined on: [-1, 1] of the inner box maps linearly, everything
// outside is folded into (1, 2) per axis, then (c + 2) / 4.  modules/NeRF/processRays.cu:21-46.
__device__ __forceinline__ float3 contract_pos(float3 pos, float3 aabb_min, float3 aabb_max) {
    const float ex = aabb_max.x - aabb_min.x, ey = aabb_max.y - aabb_min.y, ez = aabb_max.z - aabb_min.z;
    const float rx = (pos.x - aabb_min.x) / ex, ry = (pos.y - aabb_min.y) / ey, rz = (pos.z - aabb_min.z) / ez;
    const float cx = contract_axis(rx * 2.0f - 1.0f), cy = contract_axis(ry * 2.0f - 1.0f), cz = contract_axis(rz * 2.0f - 1.0f);
    return make_float3(fmaxf(0.0f, fminf((cx + 2.0f) * 0.25f, 1.0f)), fmaxf(0.0f, fminf((cy + 2.0f) * 0.25f, 1.0f)),
                       fmaxf(0.0f, fminf((cz + 2.0f) * 0.25f, 1.0f)));
}


}  // namespace nb
