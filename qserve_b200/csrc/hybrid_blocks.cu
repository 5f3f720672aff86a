// qserve_b200 -- building blocks of the hybrid decoders around the mixers: several residual streams with learned read / write / mixing
// coefficients (hyper-connections) and a group-wise RMS norm, the mean of two normed branches, query / key preparation with biases and
// unit-RMS heads, and the router and activation of a mixture-of-experts feed-forward.  The flat token batch is described in hybrid.cu.
#include <cuda_bf16.h>
#include <math.h>

#include <algorithm>

#include "../../include/qserve_b200.h"
#include "common.cuh"
#include "hybrid_common.cuh"
#include "launch.h"

namespace qs {
namespace {

using namespace hyb;

constexpr int kMaxStreams = 16;

// ---------------------------------------------------------------------------------------------------------------------------------
// Residual streams x [tokens][S][W] fp32.  One block per token:
//   1. (upd != null) the pending write of the previous sublayer, all streams at once from the old ones:
//        x_t <- sum_s mix[s][t] x_s + cout[t] y          (y: the sublayer's output row, fp32 or storage type)
//   2. u = sum_s cin[s] x_s                              (cin == null: the plain sum)
//   3. (out_sum != null) out_sum <- u   (fp32)
//   4. (out_h != null) out_h <- u, brought to unit RMS in `groups` equal consecutive parts, times (offset + w)
// With S = 1, mix = cout = cin = {1} this is the usual residual add followed by a norm.
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename ST>
__global__ void stream_norm_kernel(ST* __restrict__ out_h, float* __restrict__ out_sum, float* __restrict__ x, int S, const void* __restrict__ upd,
                                   int upd_f32, const float* __restrict__ mix, const float* __restrict__ cout, const float* __restrict__ cin,
                                   const float* __restrict__ w, int groups, float offset, float eps, int W) {
  extern __shared__ float dyn[];  // u [W] | partial sums [groups * per] | 1 / rms [groups]
  __shared__ float c_mix[kMaxStreams * kMaxStreams], c_out[kMaxStreams], c_in[kMaxStreams];
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
  for (int i = tid; i < S * S; i += blockDim.x) c_mix[i] = upd != nullptr ? mix[i] : 0.f;
  for (int i = tid; i < S; i += blockDim.x) {
    c_out[i] = upd != nullptr ? cout[i] : 0.f;
    c_in[i] = cin != nullptr ? cin[i] : 1.f;
  }
  __syncthreads();
  float* u_s = dyn;
  float* xr = x + (size_t)t * S * W;
  for (int i = tid; i < W; i += blockDim.x) {
    float xs[kMaxStreams];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s) xs[s] = s < S ? xr[(size_t)s * W + i] : 0.f;
    if (upd != nullptr) {
      const float y = upd_f32 ? static_cast<const float*>(upd)[(size_t)t * W + i] : ldf(static_cast<const ST*>(upd) + (size_t)t * W + i);
      float nx[kMaxStreams];
#pragma unroll
      for (int d = 0; d < kMaxStreams; ++d) {
        if (d < S) {
          float a = 0.f;
#pragma unroll
          for (int s = 0; s < kMaxStreams; ++s)
            if (s < S) a += c_mix[s * S + d] * xs[s];
          nx[d] = a + c_out[d] * y;
        }
      }
#pragma unroll
      for (int d = 0; d < kMaxStreams; ++d)
        if (d < S) {
          xs[d] = nx[d];
          xr[(size_t)d * W + i] = nx[d];
        }
    }
    float u = 0.f;
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s)
      if (s < S) u += c_in[s] * xs[s];
    u_s[i] = u;
    if (out_sum != nullptr) out_sum[(size_t)t * W + i] = u;
  }
  if (out_h == nullptr) return;
  __syncthreads();
  // sums of squares: `per` warps share a group, each over its own slice; the slices' sums are added in a fixed order
  const int part = W / groups, per = max(1, nw / groups), units = groups * per, len = (part + per - 1) / per;
  float* partial = dyn + W;
  float* rinv = partial + units;
  for (int un = warp; un < units; un += nw) {
    const int g = un / per, sub = un - g * per;
    const int lo = sub * len, hi = min(part, lo + len);
    float ss = 0.f;
    for (int i = lo + lane; i < hi; i += 32) {
      const float v = u_s[g * part + i];
      ss += v * v;
    }
    ss = warp_sum(ss);
    if (lane == 0) partial[un] = ss;
  }
  __syncthreads();
  for (int g = tid; g < groups; g += blockDim.x) {
    float ss = 0.f;
    for (int sub = 0; sub < per; ++sub) ss += partial[g * per + sub];
    rinv[g] = 1.f / sqrtf(ss / (float)part + eps);
  }
  __syncthreads();
  for (int i = tid; i < W; i += blockDim.x) stf(out_h + (size_t)t * W + i, u_s[i] * rinv[i / part] * (offset + w[i]));
}

// the same for widths that are multiples of 4 and 16-byte aligned rows: four columns per thread, the stream count a compile-time constant
template <typename ST, int S>
__global__ void stream_norm_vec_kernel(ST* __restrict__ out_h, float* __restrict__ out_sum, float* __restrict__ x, const void* __restrict__ upd,
                                       int upd_f32, const float* __restrict__ mix, const float* __restrict__ cout, const float* __restrict__ cin,
                                       const float* __restrict__ w, int groups, float offset, float eps, int W) {
  extern __shared__ __align__(16) float dyn[];  // u [W] | partial sums [groups * per] | 1 / rms [groups]
  __shared__ float c_mix[S * S], c_out[S], c_in[S];
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
  for (int i = tid; i < S * S; i += blockDim.x) c_mix[i] = upd != nullptr ? mix[i] : 0.f;
  for (int i = tid; i < S; i += blockDim.x) {
    c_out[i] = upd != nullptr ? cout[i] : 0.f;
    c_in[i] = cin != nullptr ? cin[i] : 1.f;
  }
  __syncthreads();
  float* u_s = dyn;
  float* xr = x + (size_t)t * S * W;
  for (int i = tid * 4; i < W; i += blockDim.x * 4) {
    float4 xs[S];
#pragma unroll
    for (int s = 0; s < S; ++s) xs[s] = ld4(xr + (size_t)s * W + i);
    if (upd != nullptr) {
      const float4 y = upd_f32 ? ld4(static_cast<const float*>(upd) + (size_t)t * W + i) : ld4(static_cast<const ST*>(upd) + (size_t)t * W + i);
      float4 nx[S];
#pragma unroll
      for (int d = 0; d < S; ++d) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < S; ++s) {
          const float m = c_mix[s * S + d];
          a.x += m * xs[s].x; a.y += m * xs[s].y; a.z += m * xs[s].z; a.w += m * xs[s].w;
        }
        const float o = c_out[d];
        nx[d] = make_float4(a.x + o * y.x, a.y + o * y.y, a.z + o * y.z, a.w + o * y.w);
      }
#pragma unroll
      for (int d = 0; d < S; ++d) {
        xs[d] = nx[d];
        st4(xr + (size_t)d * W + i, nx[d]);
      }
    }
    float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < S; ++s) {
      const float c = c_in[s];
      u.x += c * xs[s].x; u.y += c * xs[s].y; u.z += c * xs[s].z; u.w += c * xs[s].w;
    }
    *reinterpret_cast<float4*>(u_s + i) = u;
    if (out_sum != nullptr) st4(out_sum + (size_t)t * W + i, u);
  }
  if (out_h == nullptr) return;
  __syncthreads();
  const int part = W / groups, per = max(1, nw / groups), units = groups * per, len = (part + per - 1) / per;
  float* partial = dyn + W;
  float* rinv = partial + units;
  for (int un = warp; un < units; un += nw) {
    const int g = un / per, sub = un - g * per;
    const int lo = sub * len, hi = min(part, lo + len);
    float ss = 0.f;
    for (int i = lo + lane; i < hi; i += 32) {
      const float v = u_s[g * part + i];
      ss += v * v;
    }
    ss = warp_sum(ss);
    if (lane == 0) partial[un] = ss;
  }
  __syncthreads();
  for (int g = tid; g < groups; g += blockDim.x) {
    float ss = 0.f;
    for (int sub = 0; sub < per; ++sub) ss += partial[g * per + sub];
    rinv[g] = 1.f / sqrtf(ss / (float)part + eps);
  }
  __syncthreads();
  for (int i = tid * 4; i < W; i += blockDim.x * 4) {
    const float4 u = *reinterpret_cast<const float4*>(u_s + i), g = ld4(w + i);
    st4(out_h + (size_t)t * W + i, make_float4(u.x * rinv[i / part] * (offset + g.x), u.y * rinv[(i + 1) / part] * (offset + g.y),
                                               u.z * rinv[(i + 2) / part] * (offset + g.z), u.w * rinv[(i + 3) / part] * (offset + g.w)));
  }
}

// y = scale * (a * rsqrt(mean(a^2) + eps) * wa + b * rsqrt(mean(b^2) + eps) * wb): two branches, each normed over the whole row with its own
// gain; y fp32
template <typename ST>
__global__ void branch_norm_mean_kernel(float* __restrict__ y, const ST* __restrict__ a, const ST* __restrict__ b, const float* __restrict__ wa,
                                        const float* __restrict__ wb, float scale, float eps, int W) {
  __shared__ float red[33];
  const size_t base = (size_t)blockIdx.x * W;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float va = ldf(a + base + i), vb = ldf(b + base + i);
    sa += va * va;
    sb += vb * vb;
  }
  sa = block_sum(sa, red);
  sb = block_sum(sb, red);
  const float ra = 1.f / sqrtf(sa / (float)W + eps), rb = 1.f / sqrtf(sb / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) y[base + i] = scale * (ldf(a + base + i) * ra * wa[i] + ldf(b + base + i) * rb * wb[i]);
}

// the same for widths that are multiples of 4 and 16-byte aligned rows
template <typename ST>
__global__ void branch_norm_mean_vec_kernel(float* __restrict__ y, const ST* __restrict__ a, const ST* __restrict__ b, const float* __restrict__ wa,
                                            const float* __restrict__ wb, float scale, float eps, int W) {
  __shared__ float red[33];
  const size_t base = (size_t)blockIdx.x * W;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
    const float4 va = ld4(a + base + i), vb = ld4(b + base + i);
    sa += va.x * va.x + va.y * va.y + va.z * va.z + va.w * va.w;
    sb += vb.x * vb.x + vb.y * vb.y + vb.z * vb.z + vb.w * vb.w;
  }
  sa = block_sum(sa, red);
  sb = block_sum(sb, red);
  const float ra = scale / sqrtf(sa / (float)W + eps), rb = scale / sqrtf(sb / (float)W + eps);
  for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
    const float4 va = ld4(a + base + i), vb = ld4(b + base + i), ga = ld4(wa + i), gb = ld4(wb + i);
    st4(y + base + i, make_float4(va.x * ra * ga.x + vb.x * rb * gb.x, va.y * ra * ga.y + vb.y * rb * gb.y, va.z * ra * ga.z + vb.z * rb * gb.z,
                                  va.w * ra * ga.w + vb.w * rb * gb.w));
  }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// Query / key preparation of an attention layer and the append to the paged cache (one softmax map per head).
//   projection row: [H*D q | G*D k | G*Dv v];  bias (fp32, same layout) may be null
//   per head, in this order: + bias;  (unit_rms) x <- x * rsqrt(mean(x^2) + eps) [* q_gain or k_gain, fp32 [D] shared by the heads];  rotary
//   on the first rot_dims entries (layout 0: pairs (2i, 2i+1), layout 1: pairs (i, i + rot_dims/2); angle = position * inv_freq[i]);  queries
//   times q_factor[head] (may be null).  tied_values: the row has no v part, a key head's value is that key head as projected (+ bias), not yet normed.
// grid (tokens, H + G): the first H blocks finish a query head in place, the others store a key head and its value head (+ bias) in the pages
// K [page][page_size][G][D], V [page][page_size][G][Dv].
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename ST>
__global__ void qk_prepare_append_kernel(ST* __restrict__ proj, long long stride, const float* __restrict__ bias, const float* __restrict__ q_factor,
                                         const int* __restrict__ tok_slot, const int* __restrict__ tok_pos, const int* __restrict__ block_table,
                                         int max_blocks, ST* __restrict__ kpool, ST* __restrict__ vpool, const float* __restrict__ inv_freq,
                                         int rot_layout, int rot_dims, int unit_rms, float eps, int H, int G, int D, int Dv, int page,
                                         const float* __restrict__ q_gain, const float* __restrict__ k_gain, int tied_values) {
  extern __shared__ float hs[];  // the head, D floats
  __shared__ float red[33];
  const int t = blockIdx.x, u = blockIdx.y;
  const int pos = tok_pos[t];
  ST* row = proj + (size_t)t * stride;
  const bool is_q = u < H;
  const int g = u - H;
  const size_t c0 = is_q ? (size_t)u * D : (size_t)H * D + (size_t)g * D;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float v = ldf(row + c0 + i) + (bias != nullptr ? bias[c0 + i] : 0.f);
    hs[i] = v;
    ss += v * v;
  }
  float r = 1.f;
  if (unit_rms) {
    ss = block_sum(ss, red);
    r = 1.f / sqrtf(ss / (float)D + eps);
  } else {
    __syncthreads();
  }
  const float f = is_q && q_factor != nullptr ? q_factor[u] : 1.f;
  ST* dst = row + c0;
  if (!is_q) {
    const int pg = block_table[(size_t)tok_slot[t] * max_blocks + pos / page];
    const size_t cell = (size_t)pg * page + (pos % page);
    dst = kpool + (cell * G + g) * (size_t)D;
    const size_t v0 = (size_t)(H + G) * D + (size_t)g * Dv;
    ST* vd = vpool + (cell * G + g) * (size_t)Dv;
    if (tied_values) {
      for (int i = threadIdx.x; i < D; i += blockDim.x) stf(vd + i, hs[i]);
    } else {
      for (int i = threadIdx.x; i < Dv; i += blockDim.x) stf(vd + i, ldf(row + v0 + i) + (bias != nullptr ? bias[v0 + i] : 0.f));
    }
  }
  const float* gain = is_q ? q_gain : k_gain;
  if (gain != nullptr) {
    __syncthreads();  // the values above read the head as projected
    for (int i = threadIdx.x; i < D; i += blockDim.x) hs[i] *= gain[i];
    __syncthreads();
  }
  const int half = rot_dims >> 1;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float v = hs[i] * r;
    if (i < rot_dims) {
      int p, other;
      bool first;
      if (rot_layout == 0) { p = i >> 1; first = (i & 1) == 0; other = i ^ 1; }
      else { first = i < half; p = first ? i : i - half; other = first ? i + half : i - half; }
      float sn, cs;
      sincosf((float)pos * inv_freq[p], &sn, &cs);
      const float o = hs[other] * r;
      v = first ? v * cs - o * sn : v * cs + o * sn;
    }
    stf(dst + i, v * f);
  }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// Router of a mixture of experts: fp32 logits z = W_r h, scores = softmax(z) over all experts, the `top` largest scores are kept (ties: the
// lower index) as they are (no renormalisation).  One block per token; a warp per expert for the dot products.
//   route [tokens][E] fp32: the score of a chosen expert, 0 elsewhere;   top_idx / top_w [tokens][top]: the chosen experts, best first
// ---------------------------------------------------------------------------------------------------------------------------------
constexpr int kRouterEPW = 4;

// Grouped sigmoid routing of one token by one warp.  zk [3 E]: logits in, then choice scores | scores | group scores.
//   s_e = sigmoid(z_e); choice c_e = s_e + correction_e; experts form `groups` equal runs of neighbours, a group's score is the sum of its two
//   largest choice scores (its only one, for groups of one); only experts of the `keep` best groups can be chosen (ties: the lower index);
//   the `top` largest choices win, weighted with s_e / (sum of the winners' s + 1e-20).
__device__ __forceinline__ void route_sigmoid_groups(float* __restrict__ zk, float* __restrict__ route_t, int* __restrict__ idx_t, float* __restrict__ w_t,
                                                     const float* __restrict__ correction, int E, int top, int groups, int keep, int lane) {
  float* sc = zk + E;
  float* gs = zk + 2 * E;
  const int per = E / groups;
  for (int e = lane; e < E; e += 32) {
    const float s = 1.f / (1.f + expf(-zk[e]));
    sc[e] = s;
    zk[e] = s + (correction != nullptr ? correction[e] : 0.f);
    route_t[e] = 0.f;
  }
  __syncwarp();
  if (keep < groups) {
    for (int g = lane; g < groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;  // largest, second largest
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float v = zk[e];
        if (v > a) { b = a; a = v; }
        else if (v > b) b = v;
      }
      gs[g] = per > 1 ? a + b : a;
    }
    __syncwarp();
    // the groups that are not kept: all but the `keep` best; a kept group is marked by +inf
    for (int j = 0; j < keep; ++j) {
      float best = -INFINITY;
      int bi = groups;
      for (int g = lane; g < groups; g += 32)
        if (gs[g] != INFINITY && (bi == groups || gs[g] > best)) { best = gs[g]; bi = g; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi < groups && (bi == groups || ob > best || (ob == best && oi < bi))) { best = ob; bi = oi; }
      }
      if (lane == 0 && bi < groups) gs[bi] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gs[e / per] != INFINITY) zk[e] = -INFINITY;
    __syncwarp();
  }
  float total = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int bi = E;
    for (int e = lane; e < E; e += 32)
      if (!isnan(zk[e]) && (bi == E || zk[e] > best)) { best = zk[e]; bi = e; }  // NaN marks a taken expert
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi < E && (bi == E || ob > best || (ob == best && oi < bi))) { best = ob; bi = oi; }
    }
    if (bi >= E) bi = 0;  // cannot happen while top <= experts
    total += sc[bi];
    if (lane == 0) {
      idx_t[j] = bi;
      zk[bi] = __int_as_float(0x7fc00000);
    }
    __syncwarp();
  }
  const float inv = 1.f / (total + 1e-20f);
  if (lane == 0)
    for (int j = 0; j < top; ++j) {
      const float wv = sc[idx_t[j]] * inv;
      w_t[j] = wv;
      route_t[idx_t[j]] = wv;
    }
}

template <typename ST, int TOK>
__global__ void __launch_bounds__(256) moe_router_kernel(float* __restrict__ route, int* __restrict__ top_idx, float* __restrict__ top_w,
                                                         const ST* __restrict__ h, const float* __restrict__ w_router, int T, int W, int E, int top,
                                                         int zs, int mode, const float* __restrict__ correction, int groups, int keep) {
  // TOK tokens per block (rows h [TOK][W] in shared memory, storage type) and kRouterEPW experts per warp: a router word read from global
  // memory meets TOK rows, a row word read from shared memory meets kRouterEPW experts.  The dot product of a (token, expert) pair is summed
  // in the same order (lane-strided partial sums, then a shuffle tree) whatever else the block holds.  Scores [TOK][E] follow the rows.
  extern __shared__ __align__(16) unsigned char dyn_raw[];
  ST* hs = reinterpret_cast<ST*>(dyn_raw);
  float* z = reinterpret_cast<float*>(dyn_raw + (((size_t)TOK * W * sizeof(ST) + 15) & ~(size_t)15));
  const int t0 = blockIdx.x * TOK, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
  const int nt = min(TOK, T - t0);
  for (int i = tid; i < nt * W; i += blockDim.x) hs[i] = h[(size_t)t0 * W + i];
  for (int i = nt * W + tid; i < TOK * W; i += blockDim.x) stf(hs + i, 0.f);
  __syncthreads();
  for (int e0 = warp * kRouterEPW; e0 < E; e0 += nw * kRouterEPW) {
    const float* wr[kRouterEPW];
#pragma unroll
    for (int j = 0; j < kRouterEPW; ++j) wr[j] = w_router + (size_t)min(e0 + j, E - 1) * W;  // experts past the last repeat it and are dropped
    float d[kRouterEPW][TOK];
#pragma unroll
    for (int j = 0; j < kRouterEPW; ++j)
#pragma unroll
      for (int k = 0; k < TOK; ++k) d[j][k] = 0.f;
    for (int i = lane; i < W; i += 32) {
      float hv[TOK];
#pragma unroll
      for (int k = 0; k < TOK; ++k) hv[k] = ldf(hs + k * W + i);
#pragma unroll
      for (int j = 0; j < kRouterEPW; ++j) {
        const float wv = wr[j][i];
#pragma unroll
        for (int k = 0; k < TOK; ++k) d[j][k] += hv[k] * wv;
      }
    }
#pragma unroll
    for (int j = 0; j < kRouterEPW; ++j)
#pragma unroll
      for (int k = 0; k < TOK; ++k) {
        const float v = warp_sum(d[j][k]);
        if (lane == 0 && e0 + j < E) z[k * zs + e0 + j] = v;
      }
  }
  __syncthreads();
  for (int k = warp; k < nt; k += nw) {  // a warp finishes a token: softmax over all experts, then the `top` largest one by one
    const size_t t = t0 + k;
    float* zk = z + k * zs;
    if (mode == 1) {
      route_sigmoid_groups(zk, route + t * E, top_idx + t * top, top_w + t * top, correction, E, top, groups, keep, lane);
      continue;
    }
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, zk[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(zk[e] - mx);
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int e = lane; e < E; e += 32) {
      zk[e] = expf(zk[e] - mx) * inv;
      route[t * E + e] = 0.f;
    }
    __syncwarp();
    for (int j = 0; j < top; ++j) {
      float best = -1.f;
      int bi = E;
      for (int e = lane; e < E; e += 32)
        if (zk[e] > best) { best = zk[e]; bi = e; }  // strict: the lowest index of a lane's equal scores stays
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      if (lane == 0) {
        route[t * E + bi] = best;
        top_idx[t * top + j] = bi;
        top_w[t * top + j] = best;
        zk[bi] = -1.f;  // scores are positive: taken
      }
      __syncwarp();
    }
  }
}

// Activation of all experts of a token at once.  in row: [F gate | F up] with F = E * ff + ff_shared columns, expert e's at [e ff, (e + 1) ff),
// the shared expert's last.  g = min(gate, limit), u = clamp(up, -limit, limit), act = g sigmoid(alpha g) (u + shift)  (limit = +inf, alpha = 1, shift = 0: silu(gate) up);
// out[t][j] = route[t][expert of j] * act (shared columns: weight 1).  An expert that the token does not use contributes exact zeros.
template <typename ST>
__global__ void moe_act_kernel(ST* __restrict__ out, const ST* __restrict__ in, const float* __restrict__ route, int E, int ff, float limit,
                               int ff_shared, float limit_shared, float alpha, float shift) {
  const int t = blockIdx.x;
  const int F = E * ff + ff_shared;
  const int j = blockIdx.y * blockDim.x + threadIdx.x;
  if (j >= F) return;
  float wgt = 1.f, lim = limit_shared;
  if (j < E * ff) {
    wgt = route[(size_t)t * E + j / ff];
    lim = limit;
  }
  float y = 0.f;
  if (wgt != 0.f) {
    const float g = fminf(ldf(in + (size_t)t * 2 * F + j), lim);
    const float u = fminf(fmaxf(ldf(in + (size_t)t * 2 * F + F + j), -lim), lim);
    y = wgt * (g / (1.f + expf(-alpha * g))) * (u + shift);
  }
  stf(out + (size_t)t * F + j, y);
}

// bfloat16 rows, eight columns per thread (expert sizes that are multiples of 8: a thread's columns belong to one expert).
// sigmoid(alpha g) = 1 / (1 + 2^(-alpha g log2 e)): one exponential and one division on the special-function unit, far below the rounding of
// the bfloat16 result
__global__ void moe_act_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ in, const float* __restrict__ route, int E,
                                      int ff, float limit, int ff_shared, float limit_shared, float alpha, float shift) {
  const int t = blockIdx.x;
  const int F = E * ff + ff_shared;
  const int j = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (j >= F) return;
  float wgt = 1.f, lim = limit_shared;
  if (j < E * ff) {
    wgt = route[(size_t)t * E + j / ff];
    lim = limit;
  }
  __nv_bfloat16* o = out + (size_t)t * F + j;
  if (wgt == 0.f) {
    *reinterpret_cast<uint4*>(o) = make_uint4(0, 0, 0, 0);
    return;
  }
  const __nv_bfloat16* row = in + (size_t)t * 2 * F;
  const float4 g0 = ld4(row + j), g1 = ld4(row + j + 4), u0 = ld4(row + F + j), u1 = ld4(row + F + j + 4);
  const float na = -alpha * 1.4426950408889634f;
  auto f = [&](float g, float u) {
    g = fminf(g, lim);
    u = fminf(fmaxf(u, -lim), lim);
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(na * g));
    return wgt * __fdividef(g, 1.f + e) * (u + shift);
  };
  st4(o, make_float4(f(g0.x, u0.x), f(g0.y, u0.y), f(g0.z, u0.z), f(g0.w, u0.w)));
  st4(o + 4, make_float4(f(g1.x, u1.x), f(g1.y, u1.y), f(g1.z, u1.z), f(g1.w, u1.w)));
}

// ---------------------------------------------------------------------------------------------------------------------------------
// Expert-sorted rows.  Entry i = token * top + choice of top_idx names an expert; the entries of expert 0 come first, then expert 1's, ...,
// each expert's in token order (so the order never depends on timing).  Two kernels, one block per expert:
//   count: how many entries of the expert each thread's contiguous chunk of entries holds, and their sum
//   place: row_of[i] = the entry's row in the sorted order, src_token[row] = its token, ends[e] = one past the expert's last row
// ---------------------------------------------------------------------------------------------------------------------------------
constexpr int kPlanThreads = 256;

__global__ void __launch_bounds__(kPlanThreads) moe_count_kernel(int* __restrict__ counts, int* __restrict__ chunk_counts,
                                                                 const int* __restrict__ top_idx, int n) {
  __shared__ int red[kPlanThreads / 32];
  const int e = blockIdx.x, tid = threadIdx.x;
  const int per = (n + kPlanThreads - 1) / kPlanThreads, lo = tid * per, hi = min(n, lo + per);
  int c = 0;
  for (int i = lo; i < hi; ++i) c += top_idx[i] == e;
  chunk_counts[e * kPlanThreads + tid] = c;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((tid & 31) == 0) red[tid >> 5] = c;
  __syncthreads();
  if (tid == 0) {
    int t = 0;
    for (int w = 0; w < kPlanThreads / 32; ++w) t += red[w];
    counts[e] = t;
  }
}

__global__ void __launch_bounds__(kPlanThreads) moe_place_kernel(int* __restrict__ ends, int* __restrict__ row_of, int* __restrict__ src_token,
                                                                 const int* __restrict__ counts, const int* __restrict__ chunk_counts,
                                                                 const int* __restrict__ top_idx, int n, int top) {
  __shared__ int scan[kPlanThreads];
  __shared__ int base_s;
  const int e = blockIdx.x, tid = threadIdx.x;
  const int mine = chunk_counts[e * kPlanThreads + tid];
  scan[tid] = mine;
  if (tid == 0) {
    int b = 0;
    for (int i = 0; i < e; ++i) b += counts[i];
    base_s = b;
    ends[e] = b + counts[e];
  }
  __syncthreads();
  for (int o = 1; o < kPlanThreads; o <<= 1) {  // inclusive scan of the chunks' counts
    const int v = tid >= o ? scan[tid - o] : 0;
    __syncthreads();
    scan[tid] += v;
    __syncthreads();
  }
  int pos = base_s + scan[tid] - mine;
  const int per = (n + kPlanThreads - 1) / kPlanThreads, lo = tid * per, hi = min(n, lo + per);
  for (int i = lo; i < hi; ++i)
    if (top_idx[i] == e) {
      row_of[i] = pos;
      src_token[pos] = i / top;
      ++pos;
    }
}

// xs[row] = h[src_token[row]]
template <typename ST>
__global__ void moe_gather_kernel(ST* __restrict__ xs, const ST* __restrict__ h, const int* __restrict__ src_token, int W, int vec) {
  const size_t r = blockIdx.x, t = src_token[r];
  if (vec) {
    const int n16 = W * (int)sizeof(ST) / 16;
    const uint4* src = reinterpret_cast<const uint4*>(h + t * W);
    uint4* dst = reinterpret_cast<uint4*>(xs + r * W);
    for (int i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = src[i];
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) xs[r * W + i] = h[t * W + i];
  }
}

// y[t] = shared[t] + sum_k top_w[t][k] * rows[row_of[t * top + k]]   (fp32 sums in the order of k; y fp32; shared may be null)
template <typename ST>
__global__ void moe_combine_kernel(float* __restrict__ y, const ST* __restrict__ rows, const ST* __restrict__ shared, const int* __restrict__ row_of,
                                   const float* __restrict__ top_w, int top, int W) {
  const size_t t = blockIdx.x;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float a = shared != nullptr ? ldf(shared + t * W + i) : 0.f;
    for (int k = 0; k < top; ++k) a += top_w[t * top + k] * ldf(rows + (size_t)row_of[t * top + k] * W + i);
    y[t * W + i] = a;
  }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// Residual update and norm of a plain fp32 stream x [tokens][W].  One block per token:
//   1. x <- x + add1 + add2 + add_bias      (each may be null; add1 / add2 rows are fp32 or of the storage type, add_bias fp32 [W])
//   2. (cat_out != null) cat_out[t] <- [x | x0[t]]  in the storage type (the input row of a projection of the stream beside another stream)
//   3. (out_h != null) kind 1: out_h <- x * rsqrt(mean(x^2) + eps) * w
//                      kind 2: out_h <- (x - mean) * rsqrt(mean((x - mean)^2) + eps) * w + b       (two passes: mean, then deviations)
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename ST>
__global__ void stream_update_norm_kernel(ST* __restrict__ out_h, ST* __restrict__ cat_out, float* __restrict__ x, const float* __restrict__ x0,
                                          const void* __restrict__ add1, int add1_f32, const void* __restrict__ add2, int add2_f32,
                                          const float* __restrict__ add_bias, const float* __restrict__ w, const float* __restrict__ b, int kind,
                                          float eps, int W) {
  __shared__ float red[33];
  const size_t base = (size_t)blockIdx.x * W;
  float* row = x + base;
  float sum = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = row[i];
    if (add1 != nullptr || add2 != nullptr || add_bias != nullptr) {
      float u = 0.f;  // the sublayers' outputs are summed first, then meet the stream
      if (add1 != nullptr) u += add1_f32 ? static_cast<const float*>(add1)[base + i] : ldf(static_cast<const ST*>(add1) + base + i);
      if (add2 != nullptr) u += add2_f32 ? static_cast<const float*>(add2)[base + i] : ldf(static_cast<const ST*>(add2) + base + i);
      if (add_bias != nullptr) u += add_bias[i];
      v += u;
      row[i] = v;
    }
    if (cat_out != nullptr) {
      stf(cat_out + 2 * base + i, v);
      stf(cat_out + 2 * base + W + i, x0[base + i]);
    }
    sum += kind == 2 ? v : v * v;
  }
  if (out_h == nullptr) return;
  sum = block_sum(sum, red);
  float mean = 0.f, r;
  if (kind == 2) {
    mean = sum / (float)W;
    float ss = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {  // each thread re-reads what it wrote itself
      const float d = row[i] - mean;
      ss += d * d;
    }
    ss = block_sum(ss, red);
    r = 1.f / sqrtf(ss / (float)W + eps);
  } else {
    r = 1.f / sqrtf(sum / (float)W + eps);
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = (row[i] - mean) * r * w[i];
    if (b != nullptr) v += b[i];
    stf(out_h + base + i, v);
  }
}

// the same for widths that are multiples of 4 and 16-byte aligned rows: four elements per access
template <typename ST>
__global__ void stream_update_norm_vec_kernel(ST* __restrict__ out_h, ST* __restrict__ cat_out, float* __restrict__ x, const float* __restrict__ x0,
                                              const void* __restrict__ add1, int add1_f32, const void* __restrict__ add2, int add2_f32,
                                              const float* __restrict__ add_bias, const float* __restrict__ w, const float* __restrict__ b, int kind,
                                              float eps, int W) {
  __shared__ float red[33];
  const size_t base = (size_t)blockIdx.x * W;
  const bool adds = add1 != nullptr || add2 != nullptr || add_bias != nullptr;
  auto rows4 = [&](const void* p, int f32, size_t i) {
    return f32 ? ld4(static_cast<const float*>(p) + i) : ld4(static_cast<const ST*>(p) + i);
  };
  float sum = 0.f;
  for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
    float4 v = ld4(x + base + i);
    if (adds) {
      float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
      if (add1 != nullptr) { const float4 a = rows4(add1, add1_f32, base + i); u.x += a.x; u.y += a.y; u.z += a.z; u.w += a.w; }
      if (add2 != nullptr) { const float4 a = rows4(add2, add2_f32, base + i); u.x += a.x; u.y += a.y; u.z += a.z; u.w += a.w; }
      if (add_bias != nullptr) { const float4 a = ld4(add_bias + i); u.x += a.x; u.y += a.y; u.z += a.z; u.w += a.w; }
      v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
      st4(x + base + i, v);
    }
    if (cat_out != nullptr) {
      st4(cat_out + 2 * base + i, v);
      st4(cat_out + 2 * base + W + i, ld4(x0 + base + i));
    }
    sum += kind == 2 ? (v.x + v.y) + (v.z + v.w) : v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (out_h == nullptr) return;
  sum = block_sum(sum, red);
  float mean = 0.f, r;
  if (kind == 2) {
    mean = sum / (float)W;
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {  // each thread re-reads what it wrote itself
      const float4 v = ld4(x + base + i);
      const float d0 = v.x - mean, d1 = v.y - mean, d2 = v.z - mean, d3 = v.w - mean;
      ss += d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3;
    }
    ss = block_sum(ss, red);
    r = 1.f / sqrtf(ss / (float)W + eps);
  } else {
    r = 1.f / sqrtf(sum / (float)W + eps);
  }
  for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
    const float4 v = ld4(x + base + i), g = ld4(w + i);
    float4 y = make_float4((v.x - mean) * r * g.x, (v.y - mean) * r * g.y, (v.z - mean) * r * g.z, (v.w - mean) * r * g.w);
    if (b != nullptr) {
      const float4 c = ld4(b + i);
      y.x += c.x; y.y += c.y; y.z += c.z; y.w += c.w;
    }
    st4(out_h + base + i, y);
  }
}

// out[t, i] = gelu_tanh(in[t, i] + bias[i])   (bias may be null); rows of in_stride / out_stride elements
template <typename ST>
__global__ void bias_gelu_tanh_kernel(ST* __restrict__ out, long long out_stride, const ST* __restrict__ in, long long in_stride,
                                      const float* __restrict__ bias, int ff) {
  const int t = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= ff) return;
  const float z = ldf(in + (size_t)t * in_stride + i) + (bias != nullptr ? bias[i] : 0.f);
  stf(out + (size_t)t * out_stride + i, 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))));
}

// bfloat16 rows, eight columns per thread; 0.5 (1 + tanh u) = 1 / (1 + e^(-2u)) on the special-function unit
__global__ void bias_gelu_tanh_bf16x8_kernel(__nv_bfloat16* __restrict__ out, long long out_stride, const __nv_bfloat16* __restrict__ in,
                                             long long in_stride, const float* __restrict__ bias, int ff) {
  const int t = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (i >= ff) return;
  const __nv_bfloat16* row = in + (size_t)t * in_stride;
  float4 z0 = ld4(row + i), z1 = ld4(row + i + 4);
  if (bias != nullptr) {
    const float4 b0 = ld4(bias + i), b1 = ld4(bias + i + 4);
    z0.x += b0.x; z0.y += b0.y; z0.z += b0.z; z0.w += b0.w;
    z1.x += b1.x; z1.y += b1.y; z1.z += b1.z; z1.w += b1.w;
  }
  auto f = [](float z) {
    const float a = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-2.f * 1.4426950408889634f * a));
    return __fdividef(z, 1.f + e);
  };
  st4(out + (size_t)t * out_stride + i, make_float4(f(z0.x), f(z0.y), f(z0.z), f(z0.w)));
  st4(out + (size_t)t * out_stride + i + 4, make_float4(f(z1.x), f(z1.y), f(z1.z), f(z1.w)));
}

// ---------------------------------------------------------------------------------------------------------------------------------
// Post-norm residual update (blocks whose sublayers take the un-normed stream and are normed on the way out):
//   y = add [+ add_bias];   x <- x + y * rsqrt(mean(y^2) + eps) * (offset + w) [* ls];   (out_h != null) out_h <- x in the storage type
// add: rows fp32 if add_f32, else of the storage type.  One block per token; VEC: four elements per access (width a multiple of 4, 16-byte
// aligned rows).  The sum of squares is over the sublayer's output only, in fp32.
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename ST, bool VEC>
__global__ void post_norm_update_kernel(ST* __restrict__ out_h, float* __restrict__ x, const void* __restrict__ add, int add_f32,
                                        const float* __restrict__ add_bias, const float* __restrict__ w, const float* __restrict__ ls, float offset,
                                        float eps, int W) {
  __shared__ float red[33];
  const size_t base = (size_t)blockIdx.x * W;
  constexpr int V = VEC ? 4 : 1;
  auto load = [&](int i, float (&y)[V]) {
    if (VEC) {
      float4 a = add_f32 ? ld4(static_cast<const float*>(add) + base + i) : ld4(static_cast<const ST*>(add) + base + i);
      if (add_bias != nullptr) { const float4 b = ld4(add_bias + i); a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
      y[0] = a.x; y[V > 1 ? 1 : 0] = a.y; y[V > 1 ? 2 : 0] = a.z; y[V > 1 ? 3 : 0] = a.w;
    } else {
      y[0] = (add_f32 ? static_cast<const float*>(add)[base + i] : ldf(static_cast<const ST*>(add) + base + i)) + (add_bias != nullptr ? add_bias[i] : 0.f);
    }
  };
  float ss = 0.f;
  for (int i = threadIdx.x * V; i < W; i += blockDim.x * V) {
    float y[V];
    load(i, y);
#pragma unroll
    for (int k = 0; k < V; ++k) ss += y[k] * y[k];
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x * V; i < W; i += blockDim.x * V) {
    float y[V], v[V];
    load(i, y);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float u = y[k] * r * (offset + w[i + k]);
      if (ls != nullptr) u *= ls[i + k];
      v[k] = x[base + i + k] + u;
      x[base + i + k] = v[k];
    }
    if (out_h != nullptr) {
      if (VEC) st4(out_h + base + i, make_float4(v[0], v[V > 1 ? 1 : 0], v[V > 1 ? 2 : 0], v[V > 1 ? 3 : 0]));
      else stf(out_h + base + i, v[0]);
    }
  }
}

// storage-type copy of fp32 rows (the input of a sublayer that takes the un-normed stream)
template <typename ST>
__global__ void cast_rows_kernel(ST* __restrict__ out, const float* __restrict__ x, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) stf(out + i, x[i]);
}

// out[t, i] = act(in[t, i] + bias[i]) * (in[t, ff + i] + bias[ff + i])   (bias may be null); act 0: gelu_tanh, 1: silu
template <typename ST>
__global__ void bias_gated_act_kernel(ST* __restrict__ out, long long out_stride, const ST* __restrict__ in, long long in_stride,
                                      const float* __restrict__ bias, int ff, int act) {
  const int t = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= ff) return;
  const ST* row = in + (size_t)t * in_stride;
  const float z = ldf(row + i) + (bias != nullptr ? bias[i] : 0.f), u = ldf(row + ff + i) + (bias != nullptr ? bias[ff + i] : 0.f);
  const float a = act == 1 ? silu_f(z) : 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  stf(out + (size_t)t * out_stride + i, a * u);
}

// bfloat16 rows, eight columns per thread
__global__ void bias_gated_act_bf16x8_kernel(__nv_bfloat16* __restrict__ out, long long out_stride, const __nv_bfloat16* __restrict__ in,
                                             long long in_stride, const float* __restrict__ bias, int ff, int act) {
  const int t = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (i >= ff) return;
  const __nv_bfloat16* row = in + (size_t)t * in_stride;
  float z[8], u[8];
  {
    const float4 a = ld4(row + i), b = ld4(row + i + 4), c = ld4(row + ff + i), d = ld4(row + ff + i + 4);
    z[0] = a.x; z[1] = a.y; z[2] = a.z; z[3] = a.w; z[4] = b.x; z[5] = b.y; z[6] = b.z; z[7] = b.w;
    u[0] = c.x; u[1] = c.y; u[2] = c.z; u[3] = c.w; u[4] = d.x; u[5] = d.y; u[6] = d.z; u[7] = d.w;
  }
  if (bias != nullptr) {
    const float4 a = ld4(bias + i), b = ld4(bias + i + 4), c = ld4(bias + ff + i), d = ld4(bias + ff + i + 4);
    z[0] += a.x; z[1] += a.y; z[2] += a.z; z[3] += a.w; z[4] += b.x; z[5] += b.y; z[6] += b.z; z[7] += b.w;
    u[0] += c.x; u[1] += c.y; u[2] += c.z; u[3] += c.w; u[4] += d.x; u[5] += d.y; u[6] += d.z; u[7] += d.w;
  }
  float y[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float arg = act == 1 ? z[k] : 2.f * 0.7978845608028654f * (z[k] + 0.044715f * z[k] * z[k] * z[k]);  // z sigmoid(arg) is silu or gelu_tanh
    y[k] = __fdividef(z[k], 1.f + fast_exp2(-1.4426950408889634f * arg)) * u[k];
  }
  st4(out + (size_t)t * out_stride + i, make_float4(y[0], y[1], y[2], y[3]));
  st4(out + (size_t)t * out_stride + i + 4, make_float4(y[4], y[5], y[6], y[7]));
}

// x <- cap * tanh(x / cap), fp32 in place
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

}  // namespace
}  // namespace qs

using namespace qs;

#define QS_DT(dtype, CALL_BF16, CALL_F32)                                               \
  do {                                                                                  \
    if ((dtype) == QS_DTYPE_BF16) { CALL_BF16; }                                        \
    else if ((dtype) == QS_DTYPE_F32) { CALL_F32; }                                     \
    else return set_error(qs::QS_ERR_INVALID, "dtype must be QS_DTYPE_BF16 or QS_DTYPE_F32"); \
  } while (0)

extern "C" {

int qs_hyb_stream_norm(void* out_h, float* out_sum, float* x, int streams, const void* upd, int upd_f32, const float* upd_mix, const float* upd_out,
                       const float* in_coef, const float* w, int groups, float offset, float eps, int tokens_n, int width, int dtype, void* stream) {
  QS_REQUIRE(x && (out_h == nullptr || w != nullptr), "hyb_stream_norm: null tensor");
  QS_REQUIRE(streams >= 1 && streams <= kMaxStreams, "hyb_stream_norm: 1..16 streams");
  QS_REQUIRE(upd == nullptr || (upd_mix && upd_out), "hyb_stream_norm: a pending write needs its coefficients");
  QS_REQUIRE(groups >= 1 && width % groups == 0, "hyb_stream_norm: the width must split into `groups` equal parts");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = width >= 2048 ? 256 : 128;
  const int per = std::max(1, threads / 32 / groups);
  const size_t smb = ((size_t)width + (size_t)groups * per + groups) * sizeof(float);
  QS_REQUIRE(smb <= 200 * 1024, "hyb_stream_norm: row too wide for shared memory");
#define QS_LAUNCH(ST)                                                                                                                   \
  do {                                                                                                                                  \
    if (smb > 48 * 1024) cudaFuncSetAttribute(stream_norm_kernel<ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smb);           \
    stream_norm_kernel<ST><<<tokens_n, threads, smb, s>>>((ST*)out_h, out_sum, x, streams, upd, upd_f32, upd_mix, upd_out, in_coef, w,  \
                                                         groups, offset, eps, width);                                                  \
  } while (0)
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (streams <= 8 && width % 4 == 0 && al16(out_h) && al16(out_sum) && al16(x) && al16(upd) && al16(w)) {
#define QS_VEC(ST, S)                                                                                                                        \
  do {                                                                                                                                       \
    if (smb > 48 * 1024) cudaFuncSetAttribute(stream_norm_vec_kernel<ST, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smb);         \
    stream_norm_vec_kernel<ST, S><<<tokens_n, threads, smb, s>>>((ST*)out_h, out_sum, x, upd, upd_f32, upd_mix, upd_out, in_coef, w, groups,  \
                                                                offset, eps, width);                                                        \
  } while (0)
#define QS_VEC_S(ST)                        \
  switch (streams) {                        \
    case 1: QS_VEC(ST, 1); break;           \
    case 2: QS_VEC(ST, 2); break;           \
    case 3: QS_VEC(ST, 3); break;           \
    case 4: QS_VEC(ST, 4); break;           \
    case 5: QS_VEC(ST, 5); break;           \
    case 6: QS_VEC(ST, 6); break;           \
    case 7: QS_VEC(ST, 7); break;           \
    default: QS_VEC(ST, 8); break;          \
  }
    QS_DT(dtype, QS_VEC_S(__nv_bfloat16), QS_VEC_S(float));
#undef QS_VEC_S
#undef QS_VEC
    return check_cuda(cudaGetLastError(), "hyb_stream_norm");
  }
  QS_DT(dtype, QS_LAUNCH(__nv_bfloat16), QS_LAUNCH(float));
#undef QS_LAUNCH
  return check_cuda(cudaGetLastError(), "hyb_stream_norm");
}

int qs_hyb_branch_norm_mean(float* y, const void* a, const void* b, const float* wa, const float* wb, float scale, float eps, int tokens_n,
                            int width, int dtype, void* stream) {
  QS_REQUIRE(y && a && b && wa && wb, "hyb_branch_norm_mean: null tensor");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = width >= 1024 ? 256 : 128;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (width % 4 == 0 && al16(y) && al16(a) && al16(b) && al16(wa) && al16(wb)) {
    QS_DT(dtype,
          (branch_norm_mean_vec_kernel<__nv_bfloat16><<<tokens_n, threads, 0, s>>>(y, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, wa, wb, scale, eps, width)),
          (branch_norm_mean_vec_kernel<float><<<tokens_n, threads, 0, s>>>(y, (const float*)a, (const float*)b, wa, wb, scale, eps, width)));
    return check_cuda(cudaGetLastError(), "hyb_branch_norm_mean");
  }
  QS_DT(dtype,
        (branch_norm_mean_kernel<__nv_bfloat16><<<tokens_n, threads, 0, s>>>(y, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, wa, wb, scale, eps, width)),
        (branch_norm_mean_kernel<float><<<tokens_n, threads, 0, s>>>(y, (const float*)a, (const float*)b, wa, wb, scale, eps, width)));
  return check_cuda(cudaGetLastError(), "hyb_branch_norm_mean");
}

int qs_hyb_qk_prepare_append(void* proj, int64_t stride, const float* bias, const float* q_factor, const int32_t* tok_slot, const int32_t* tok_pos,
                             const int32_t* block_table, int max_blocks, void* kpool, void* vpool, const float* inv_freq, int rot_layout,
                             int rot_dims, int unit_rms, float eps, int tokens_n, int heads, int kv_heads, int dim, int vdim, int page_size,
                             const float* q_gain, const float* k_gain, int tied_values, int dtype, void* stream) {
  QS_REQUIRE(proj && tok_slot && tok_pos && block_table && kpool && vpool, "hyb_qk_prepare_append: null tensor");
  QS_REQUIRE(!tied_values || vdim == dim, "hyb_qk_prepare_append: values tied to the keys need vdim == dim");
  QS_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dim && (rot_dims == 0 || inv_freq != nullptr) && (rot_layout == 0 || rot_layout == 1),
             "hyb_qk_prepare_append: bad rotary size or layout");
  QS_REQUIRE(kv_heads > 0 && heads % kv_heads == 0 && page_size > 0 && dim > 0 && dim <= 8192, "hyb_qk_prepare_append: bad head geometry");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(tokens_n, heads + kv_heads);
  const size_t smb = (size_t)dim * sizeof(float);
  QS_DT(dtype,
        (qk_prepare_append_kernel<__nv_bfloat16><<<grid, 64, smb, s>>>((__nv_bfloat16*)proj, stride, bias, q_factor, tok_slot, tok_pos, block_table,
                                                                        max_blocks, (__nv_bfloat16*)kpool, (__nv_bfloat16*)vpool, inv_freq, rot_layout,
                                                                        rot_dims, unit_rms, eps, heads, kv_heads, dim, vdim, page_size, q_gain, k_gain,
                                                                        tied_values)),
        (qk_prepare_append_kernel<float><<<grid, 64, smb, s>>>((float*)proj, stride, bias, q_factor, tok_slot, tok_pos, block_table, max_blocks,
                                                                (float*)kpool, (float*)vpool, inv_freq, rot_layout, rot_dims, unit_rms, eps, heads,
                                                                kv_heads, dim, vdim, page_size, q_gain, k_gain, tied_values)));
  return check_cuda(cudaGetLastError(), "hyb_qk_prepare_append");
}

int qs_hyb_moe_router(float* route, int32_t* top_idx, float* top_w, const void* h, const float* w_router, int tokens_n, int width, int experts,
                      int top, int mode, const float* correction, int groups, int keep, int dtype, void* stream) {
  QS_REQUIRE(route && top_idx && top_w && h && w_router, "hyb_moe_router: null tensor");
  QS_REQUIRE(experts >= 1 && top >= 1 && top <= experts, "hyb_moe_router: 1 <= top <= experts");
  QS_REQUIRE(mode == QS_ROUTER_SOFTMAX || mode == QS_ROUTER_SIGMOID_GROUPS, "hyb_moe_router: unknown mode");
  if (mode == QS_ROUTER_SIGMOID_GROUPS)
    QS_REQUIRE(groups >= 1 && experts % groups == 0 && keep >= 1 && keep <= groups && top <= keep * (experts / groups),
               "hyb_moe_router: groups must divide the experts, 1 <= keep <= groups, top <= experts of the kept groups");
  const int zs = mode == QS_ROUTER_SIGMOID_GROUPS ? 3 * experts : experts;  // floats of work space per token
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  // tokens per block: as many as fit beside their scores in shared memory, at most 8; few tokens (decoding) go one per block
  const size_t es = dtype == QS_DTYPE_BF16 ? 2 : 4;
  auto bytes = [&](int tk) { return (((size_t)tk * width * es + 15) & ~(size_t)15) + (size_t)tk * zs * sizeof(float); };
  int tok = tokens_n >= 512 ? 8 : 1;  // every block reads the whole router once (16 tokens per block ran slower: 64 + 16 live accumulators)
  while (tok > 1 && bytes(tok) > 100 * 1024) tok >>= 1;  // two blocks per SM
  const size_t smb = bytes(tok);
  QS_REQUIRE(smb <= 200 * 1024, "hyb_moe_router: row too wide for shared memory");
#define QS_LAUNCH(ST, TOK)                                                                                                              \
  do {                                                                                                                                  \
    if (smb > 48 * 1024) cudaFuncSetAttribute(moe_router_kernel<ST, TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smb);       \
    moe_router_kernel<ST, TOK><<<(tokens_n + TOK - 1) / TOK, 256, smb, s>>>(route, top_idx, top_w, (const ST*)h, w_router, tokens_n,   \
                                                                          width, experts, top, zs, mode, correction, groups, keep);    \
  } while (0)
#define QS_LAUNCH_T(ST)                          \
  switch (tok) {                                 \
    case 8: QS_LAUNCH(ST, 8); break;             \
    case 4: QS_LAUNCH(ST, 4); break;             \
    case 2: QS_LAUNCH(ST, 2); break;             \
    default: QS_LAUNCH(ST, 1); break;            \
  }
  QS_DT(dtype, QS_LAUNCH_T(__nv_bfloat16), QS_LAUNCH_T(float));
#undef QS_LAUNCH_T
#undef QS_LAUNCH
  return check_cuda(cudaGetLastError(), "hyb_moe_router");
}

int qs_hyb_moe_act(void* out, const void* in, const float* route, int tokens_n, int experts, int ff, float limit, int ff_shared, float limit_shared,
                   float alpha, float shift, int dtype, void* stream) {
  QS_REQUIRE(out && in && (route || experts == 0), "hyb_moe_act: null tensor");
  QS_REQUIRE(experts >= 0 && ff >= 0 && ff_shared >= 0 && experts * ff + ff_shared > 0, "hyb_moe_act: no columns");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int F = experts * ff + ff_shared;
  if (dtype == QS_DTYPE_BF16 && ff % 8 == 0 && ff_shared % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(in) & 15) == 0) {
    moe_act_bf16x8_kernel<<<dim3(tokens_n, (F / 8 + 255) / 256), 256, 0, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)in, route, experts, ff, limit,
                                                                              ff_shared, limit_shared, alpha, shift);
    return check_cuda(cudaGetLastError(), "hyb_moe_act");
  }
  dim3 grid(tokens_n, (F + 255) / 256);
  QS_DT(dtype,
        (moe_act_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)in, route, experts, ff, limit, ff_shared,
                                                             limit_shared, alpha, shift)),
        (moe_act_kernel<float><<<grid, 256, 0, s>>>((float*)out, (const float*)in, route, experts, ff, limit, ff_shared, limit_shared, alpha, shift)));
  return check_cuda(cudaGetLastError(), "hyb_moe_act");
}

int qs_hyb_moe_plan(int32_t* ends, int32_t* row_of, int32_t* src_token, int32_t* work, const int32_t* top_idx, int tokens_n, int experts, int top,
                    void* stream) {
  QS_REQUIRE(ends && row_of && src_token && work && top_idx, "hyb_moe_plan: null tensor");
  QS_REQUIRE(experts >= 1 && top >= 1 && top <= experts, "hyb_moe_plan: 1 <= top <= experts");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  int* counts = work;                 // [experts]
  int* chunk_counts = work + experts;  // [experts][kPlanThreads]
  moe_count_kernel<<<experts, kPlanThreads, 0, s>>>(counts, chunk_counts, top_idx, tokens_n * top);
  moe_place_kernel<<<experts, kPlanThreads, 0, s>>>(ends, row_of, src_token, counts, chunk_counts, top_idx, tokens_n * top, top);
  return check_cuda(cudaGetLastError(), "hyb_moe_plan");
}

int64_t qs_hyb_moe_plan_work_ints(int experts) { return (int64_t)experts * (1 + kPlanThreads); }

int qs_hyb_moe_gather(void* xs, const void* h, const int32_t* src_token, int rows, int width, int dtype, void* stream) {
  QS_REQUIRE(xs && h && src_token, "hyb_moe_gather: null tensor");
  if (rows == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t es = dtype == QS_DTYPE_BF16 ? 2 : 4;
  const int vec = (width * es) % 16 == 0 && (reinterpret_cast<uintptr_t>(xs) & 15) == 0 && (reinterpret_cast<uintptr_t>(h) & 15) == 0;
  QS_DT(dtype, (moe_gather_kernel<__nv_bfloat16><<<rows, 128, 0, s>>>((__nv_bfloat16*)xs, (const __nv_bfloat16*)h, src_token, width, vec)),
        (moe_gather_kernel<float><<<rows, 128, 0, s>>>((float*)xs, (const float*)h, src_token, width, vec)));
  return check_cuda(cudaGetLastError(), "hyb_moe_gather");
}

int qs_hyb_moe_combine(float* y, const void* rows, const void* shared, const int32_t* row_of, const float* top_w, int tokens_n, int top, int width,
                       int dtype, void* stream) {
  QS_REQUIRE(y && rows && row_of && top_w, "hyb_moe_combine: null tensor");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = width >= 1024 ? 256 : 128;
  QS_DT(dtype,
        (moe_combine_kernel<__nv_bfloat16><<<tokens_n, threads, 0, s>>>(y, (const __nv_bfloat16*)rows, (const __nv_bfloat16*)shared, row_of, top_w, top, width)),
        (moe_combine_kernel<float><<<tokens_n, threads, 0, s>>>(y, (const float*)rows, (const float*)shared, row_of, top_w, top, width)));
  return check_cuda(cudaGetLastError(), "hyb_moe_combine");
}

int qs_hyb_stream_update_norm(void* out_h, void* cat_out, float* x, const float* x0, const void* add1, int add1_f32, const void* add2, int add2_f32,
                              const float* add_bias, const float* w, const float* b, int kind, float eps, int tokens_n, int width, int dtype,
                              void* stream) {
  QS_REQUIRE(x, "hyb_stream_update_norm: null stream");
  QS_REQUIRE(out_h == nullptr || ((kind == QS_NORM_RMS || kind == QS_NORM_LAYER) && w != nullptr), "hyb_stream_update_norm: a norm needs its kind and gain");
  QS_REQUIRE(cat_out == nullptr || x0 != nullptr, "hyb_stream_update_norm: the joined row needs the second stream");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = width >= 1024 ? 256 : 128;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (width % 4 == 0 && al16(out_h) && al16(cat_out) && al16(x) && al16(x0) && al16(add1) && al16(add2) && al16(add_bias) && al16(w) && al16(b)) {
    QS_DT(dtype,
          (stream_update_norm_vec_kernel<__nv_bfloat16><<<tokens_n, threads, 0, s>>>((__nv_bfloat16*)out_h, (__nv_bfloat16*)cat_out, x, x0, add1, add1_f32,
                                                                                      add2, add2_f32, add_bias, w, b, kind, eps, width)),
          (stream_update_norm_vec_kernel<float><<<tokens_n, threads, 0, s>>>((float*)out_h, (float*)cat_out, x, x0, add1, add1_f32, add2, add2_f32, add_bias,
                                                                             w, b, kind, eps, width)));
    return check_cuda(cudaGetLastError(), "hyb_stream_update_norm");
  }
  QS_DT(dtype,
        (stream_update_norm_kernel<__nv_bfloat16><<<tokens_n, threads, 0, s>>>((__nv_bfloat16*)out_h, (__nv_bfloat16*)cat_out, x, x0, add1, add1_f32, add2,
                                                                                add2_f32, add_bias, w, b, kind, eps, width)),
        (stream_update_norm_kernel<float><<<tokens_n, threads, 0, s>>>((float*)out_h, (float*)cat_out, x, x0, add1, add1_f32, add2, add2_f32, add_bias, w, b,
                                                                       kind, eps, width)));
  return check_cuda(cudaGetLastError(), "hyb_stream_update_norm");
}

int qs_hyb_bias_gelu_tanh(void* out, int64_t out_stride, const void* in, int64_t in_stride, const float* bias, int tokens_n, int ff, int dtype,
                          void* stream) {
  QS_REQUIRE(out && in, "hyb_bias_gelu_tanh: null tensor");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (dtype == QS_DTYPE_BF16 && ff % 8 == 0 && out_stride % 8 == 0 && in_stride % 8 == 0 && al16(out) && al16(in) && al16(bias)) {
    bias_gelu_tanh_bf16x8_kernel<<<dim3(tokens_n, (ff / 8 + 255) / 256), 256, 0, s>>>((__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)in, in_stride,
                                                                                     bias, ff);
    return check_cuda(cudaGetLastError(), "hyb_bias_gelu_tanh");
  }
  dim3 grid(tokens_n, (ff + 255) / 256);
  QS_DT(dtype, (bias_gelu_tanh_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)in, in_stride, bias, ff)),
        (bias_gelu_tanh_kernel<float><<<grid, 256, 0, s>>>((float*)out, out_stride, (const float*)in, in_stride, bias, ff)));
  return check_cuda(cudaGetLastError(), "hyb_bias_gelu_tanh");
}

int qs_hyb_post_norm_update(void* out_h, float* x, const void* add, int add_f32, const float* add_bias, const float* w, const float* ls, float offset,
                            float eps, int tokens_n, int width, int dtype, void* stream) {
  QS_REQUIRE(x && add && w, "hyb_post_norm_update: null tensor");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = width >= 1024 ? 256 : 128;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (width % 4 == 0 && al16(out_h) && al16(x) && al16(add) && al16(add_bias) && al16(w) && al16(ls)) {
    QS_DT(dtype,
          (post_norm_update_kernel<__nv_bfloat16, true><<<tokens_n, threads, 0, s>>>((__nv_bfloat16*)out_h, x, add, add_f32, add_bias, w, ls, offset, eps, width)),
          (post_norm_update_kernel<float, true><<<tokens_n, threads, 0, s>>>((float*)out_h, x, add, add_f32, add_bias, w, ls, offset, eps, width)));
  } else {
    QS_DT(dtype,
          (post_norm_update_kernel<__nv_bfloat16, false><<<tokens_n, threads, 0, s>>>((__nv_bfloat16*)out_h, x, add, add_f32, add_bias, w, ls, offset, eps, width)),
          (post_norm_update_kernel<float, false><<<tokens_n, threads, 0, s>>>((float*)out_h, x, add, add_f32, add_bias, w, ls, offset, eps, width)));
  }
  return check_cuda(cudaGetLastError(), "hyb_post_norm_update");
}

int qs_hyb_cast_rows(void* out, const float* x, int64_t n, int dtype, void* stream) {
  QS_REQUIRE(out && x, "hyb_cast_rows: null tensor");
  if (n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  QS_DT(dtype, (cast_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((__nv_bfloat16*)out, x, (size_t)n)),
        (cast_rows_kernel<float><<<blocks, 256, 0, s>>>((float*)out, x, (size_t)n)));
  return check_cuda(cudaGetLastError(), "hyb_cast_rows");
}

int qs_hyb_bias_gated_act(void* out, int64_t out_stride, const void* in, int64_t in_stride, const float* bias, int tokens_n, int ff, int act, int dtype,
                          void* stream) {
  QS_REQUIRE(out && in, "hyb_bias_gated_act: null tensor");
  QS_REQUIRE(act == QS_ACT_GELU_TANH || act == QS_ACT_SILU, "hyb_bias_gated_act: unknown activation");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (dtype == QS_DTYPE_BF16 && ff % 8 == 0 && out_stride % 8 == 0 && in_stride % 8 == 0 && al16(out) && al16(in) && al16(bias)) {
    bias_gated_act_bf16x8_kernel<<<dim3(tokens_n, (ff / 8 + 255) / 256), 256, 0, s>>>((__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)in, in_stride,
                                                                                     bias, ff, act);
    return check_cuda(cudaGetLastError(), "hyb_bias_gated_act");
  }
  dim3 grid(tokens_n, (ff + 255) / 256);
  QS_DT(dtype, (bias_gated_act_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)in, in_stride, bias, ff, act)),
        (bias_gated_act_kernel<float><<<grid, 256, 0, s>>>((float*)out, out_stride, (const float*)in, in_stride, bias, ff, act)));
  return check_cuda(cudaGetLastError(), "hyb_bias_gated_act");
}

int qs_hyb_softcap(float* x, int64_t n, float cap, void* stream) {
  QS_REQUIRE(x && cap > 0.f, "hyb_softcap: null tensor or cap <= 0");
  if (n == 0) return qs::QS_OK;
  softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, (size_t)n, cap);
  return check_cuda(cudaGetLastError(), "hyb_softcap");
}

}  // extern "C"
