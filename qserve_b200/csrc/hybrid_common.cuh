// qserve_b200 -- device helpers shared by the translation units of the unquantised hybrid decoders: loads / stores of the storage type
// (bfloat16 or float) as fp32, warp and block reductions, asynchronous shared-memory copies.
#pragma once
#include <cuda_bf16.h>
#include <math.h>
#include <stdint.h>

#include "common.cuh"

namespace qs {
namespace hyb {

template <typename ST> __device__ __forceinline__ float ldf(const ST* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename ST> __device__ __forceinline__ void stf(ST* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// block-wide sum / max over up to 32 warps; `red` holds 33 floats; every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x & 31) < nw ? red[threadIdx.x & 31] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x & 31) < nw ? red[threadIdx.x & 31] : -INFINITY;
  return warp_max(t);
}

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

// four elements of the storage type at once
template <typename ST> __device__ __forceinline__ float4 ld4(const ST* p);
template <> __device__ __forceinline__ float4 ld4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 ld4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
}
template <typename ST> __device__ __forceinline__ void st4(ST* p, float4 v);
template <> __device__ __forceinline__ void st4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void st4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
}

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}

// tensor-core helpers of the bfloat16 attention kernels (mma.sync m16n8k16, fragments through ldmatrix)
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x on the special-function unit (relative error about 2^-22; -inf gives 0): the bfloat16 kernels' softmax runs in the base-2 domain
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// the leading bfloat16 terms of two fp32 numbers, packed; the numbers keep what is left
__device__ __forceinline__ uint32_t split_bf16x2(float& lo, float& hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  const uint32_t u = *reinterpret_cast<uint32_t*>(&v);
  lo -= __uint_as_float(u << 16);
  hi -= __uint_as_float(u & 0xffff0000u);
  return u;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// first position a query at `pos` sees: the start of its chunk of `chunk` positions (0: no chunks), and not further back than `window`
// positions including its own (0: no window)
__host__ __device__ __forceinline__ int first_key(int pos, int chunk, int window) {
  int f = chunk > 0 ? pos - pos % chunk : 0;
  if (window > 0) f = max(f, pos - window + 1);
  return f;
}

// With a window, the first `keep` positions of a sequence may stay visible.  A walk over tiles of KT keys that starts at tile first / KT then
// also visits the tiles that hold kept positions before it: n_pre of them, tiles 0 .. n_pre - 1; walk index i stands for tile
// i < n_pre ? i : first / KT + i - n_pre.
__host__ __device__ __forceinline__ int kept_tiles(int first, int keep, int KT) { return min((keep + KT - 1) / KT, first / KT); }
__host__ __device__ __forceinline__ bool key_visible(int kpos, int qpos, int first, int keep) { return kpos <= qpos && (kpos >= first || kpos < keep); }

// optional parts of an attention kernel (qs_attn_extra of the C interface, by value)
struct AttnExtra {
  int keep_first;
  const float* slopes;
  const void* gate;
  long long gate_stride;
};
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

}  // namespace hyb
}  // namespace qs
