// qserve_b200 -- kernels of the unquantised hybrid decoders (attention layers and recurrent layers in one stack, fp32 residual stream).
//
// Everything here works on a FLAT batch of tokens: a step of the engine brings, for every live sequence, a run of consecutive
// tokens (a portion of a prompt or one decoded token).  Per-token tables (`tok_slot`, `tok_pos`, `tok_entry`) and per-entry tables
// (`entry_start`, `entry_len`, `entry_slot`, `entry_pos0`) say where a token belongs; the paged key/value cache is addressed through a
// block table indexed by the sequence's slot.  The same kernels therefore serve whole prompts, portions and single decoded tokens, and a
// position's result does not depend on what else is in the batch.
//
// Storage type ST is bfloat16 or float (the engine's activation / cache type); scores, softmax weights, norms, rotary angles, decays,
// gates of the recurrence, the recurrent state and the residual stream are fp32 in both.
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


// ---------------------------------------------------------------------------------------------------------------------------------
// embedding: token row times `scale` (+ hashed (previous, current) pair row) -> fp32 residual stream
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename ST>
__global__ void embed_pair_kernel(float* __restrict__ out, const int* __restrict__ tokens, const int* __restrict__ prev, const ST* __restrict__ table,
                                  const ST* __restrict__ pair, int W, int buckets, long long mul_prev, long long mul_cur, float scale, int copies) {
  const int t = blockIdx.x;
  const long long tok = tokens[t];
  const ST* e = table + tok * W;
  const ST* b = nullptr;
  if (pair != nullptr) {
    const long long p = prev[t];
    const long long row = p < 0 ? buckets : (p * mul_prev + tok * mul_cur) % buckets;
    b = pair + row * W;
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = ldf(e + i) * scale + (b ? ldf(b + i) : 0.f);
    for (int c = 0; c < copies; ++c) out[((size_t)t * copies + c) * W + i] = v;  // every residual stream starts from the embedding
  }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// RMS norm of the fp32 stream with one or two gains (the two branches of a parallel layer read the same normalised row):
//   [x <- x + add;]  out_k = x * rsqrt(mean(x^2) + eps) * (offset + w_k)
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename ST>
__global__ void rms_norm2_kernel(ST* __restrict__ out1, ST* __restrict__ out2, float* __restrict__ x, const ST* __restrict__ add,
                                 const float* __restrict__ w1, const float* __restrict__ w2, float offset, float eps, int W) {
  __shared__ float red[33];
  float* row = x + (size_t)blockIdx.x * W;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = row[i];
    if (add != nullptr) {  // the previous layer's update lands in the stream here: one pass instead of two
      v += ldf(add + (size_t)blockIdx.x * W + i);
      row[i] = v;
    }
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = row[i] * r;  // each thread re-reads what it wrote itself
    stf(out1 + (size_t)blockIdx.x * W + i, v * (offset + w1[i]));
    if (out2 != nullptr) stf(out2 + (size_t)blockIdx.x * W + i, v * (offset + w2[i]));
  }
}


// the same norm for widths that are multiples of 4: 16-byte accesses to the stream and the gains, 8- or 16-byte ones to the outputs
template <typename ST>
__global__ void rms_norm2_vec_kernel(ST* __restrict__ out1, ST* __restrict__ out2, float* __restrict__ x, const ST* __restrict__ add,
                                     const float* __restrict__ w1, const float* __restrict__ w2, float offset, float eps, int W) {
  __shared__ float red[33];
  const size_t base = (size_t)blockIdx.x * W;
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
    float4 v = ld4(x + base + i);
    if (add != nullptr) {
      const float4 a = ld4(add + base + i);
      v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
      st4(x + base + i, v);
    }
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
    const float4 v = ld4(x + base + i);  // each thread re-reads what it wrote itself
    const float4 g = ld4(w1 + i);
    st4(out1 + base + i, make_float4(v.x * r * (offset + g.x), v.y * r * (offset + g.y), v.z * r * (offset + g.z), v.w * r * (offset + g.w)));
    if (out2 != nullptr) {
      const float4 h = ld4(w2 + i);
      st4(out2 + base + i, make_float4(v.x * r * (offset + h.x), v.y * r * (offset + h.y), v.z * r * (offset + h.z), v.w * r * (offset + h.w)));
    }
  }
}

// x += y  (fp32 stream, y in the storage type)
template <typename ST>
__global__ void residual_add_kernel(float* __restrict__ x, const ST* __restrict__ y, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] += ldf(y + i);
}

// out[t, i] = gelu_tanh(in[t, i]) * in[t, ff + i]
template <typename ST>
__global__ void gelu_tanh_mul_kernel(ST* __restrict__ out, long long out_stride, const ST* __restrict__ in, int ff) {
  const int t = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= ff) return;
  const float z = ldf(in + (size_t)t * 2 * ff + i), u = ldf(in + (size_t)t * 2 * ff + ff + i);
  const float g = 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  stf(out + (size_t)t * out_stride + i, g * u);
}

// bfloat16 rows, eight elements per thread.  0.5 (1 + tanh u) = 1 / (1 + e^(-2u)): one exponential and one division on the special-function
// unit, relative error near 2^-21, far below the rounding of the bfloat16 result (the fp32 kernel above keeps tanhf)
__global__ void gelu_tanh_mul_bf16x8_kernel(__nv_bfloat16* __restrict__ out, long long out_stride, const __nv_bfloat16* __restrict__ in, int ff) {
  const int t = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (i >= ff) return;
  const __nv_bfloat16* row = in + (size_t)t * 2 * ff;
  const float4 z0 = ld4(row + i), z1 = ld4(row + i + 4), u0 = ld4(row + ff + i), u1 = ld4(row + ff + i + 4);
  auto f = [](float z, float u) {
    const float a = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-2.f * 1.4426950408889634f * a));
    return __fdividef(z, 1.f + e) * u;
  };
  st4(out + (size_t)t * out_stride + i, make_float4(f(z0.x, u0.x), f(z0.y, u0.y), f(z0.z, u0.z), f(z0.w, u0.w)));
  st4(out + (size_t)t * out_stride + i + 4, make_float4(f(z1.x, u1.x), f(z1.y, u1.y), f(z1.z, u1.z), f(z1.w, u1.w)));
}

// ---------------------------------------------------------------------------------------------------------------------------------
// rotary embedding (interleaved pairs, per-pair frequency table, amplitude factor) on the q and k parts of the projection row, and the
// append of the rotated key row and the value row to the paged cache.
//   row layout: [H * maps * D queries | G * maps * D keys | G * Dv values]
//   K page: [page_size][G][maps * D], V page: [page_size][G][Dv]
// grid (tokens, H + G); the first H blocks rotate a query head in place, the others rotate + store a key head and copy its value head.
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename ST>
__global__ void rope_append_kernel(ST* __restrict__ proj, long long stride, const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
                                   const int* __restrict__ block_table, int max_blocks, ST* __restrict__ kpool, ST* __restrict__ vpool,
                                   const float* __restrict__ inv_freq, float amp, int H, int G, int maps, int D, int Dv, int rot_dims, int page) {
  const int t = blockIdx.x, u = blockIdx.y;
  const int pos = tok_pos[t];
  const int half = rot_dims >> 1;
  ST* row = proj + (size_t)t * stride;
  if (u < H) {
    ST* q = row + (size_t)u * maps * D;
    for (int i = threadIdx.x; i < maps * half; i += blockDim.x) {
      const int m = i / half, p = i - m * half;
      float s, c;
      sincosf((float)pos * inv_freq[p], &s, &c);
      s *= amp; c *= amp;
      ST* a = q + m * D + 2 * p;
      const float x0 = ldf(a), x1 = ldf(a + 1);
      stf(a, x0 * c - x1 * s);
      stf(a + 1, x1 * c + x0 * s);
    }
    return;
  }
  const int g = u - H;
  const int slot = tok_slot[t];
  const int pg = block_table[(size_t)slot * max_blocks + pos / page];
  const size_t cell = (size_t)pg * page + (pos % page);
  const ST* k = row + (size_t)H * maps * D + (size_t)g * maps * D;
  ST* kd = kpool + (cell * G + g) * (size_t)(maps * D);
  for (int i = threadIdx.x; i < maps * D; i += blockDim.x) {
    const int d = i % D;
    float v;
    if (d < rot_dims) {
      const int p = d >> 1;
      float s, c;
      sincosf((float)pos * inv_freq[p], &s, &c);
      s *= amp; c *= amp;
      const int b0 = i - d;
      const float x0 = ldf(k + b0 + (d & ~1)), x1 = ldf(k + b0 + (d | 1));
      v = (d & 1) ? (x1 * c + x0 * s) : (x0 * c - x1 * s);
    } else {
      v = ldf(k + i);
    }
    stf(kd + i, v);
  }
  const ST* vs = row + (size_t)(H + G) * maps * D + (size_t)g * Dv;
  ST* vd = vpool + (cell * G + g) * (size_t)Dv;
  for (int i = threadIdx.x; i < Dv; i += blockDim.x) vd[i] = vs[i];
}

// ---------------------------------------------------------------------------------------------------------------------------------
// causal attention over the paged cache with `MAPS` softmax maps per head that share the values (MAPS = 2: differential attention).
// One block per (token, query head).  Keys are walked in tiles of KT; a warp scores one key at a time with coalesced loads of the
// key row (fp32 dot products), the block keeps an online softmax per map (fp32 weights), and thread d accumulates output dimension(s)
// d, d + blockDim, ... for every map.  Epilogue:
//   MAPS == 2: o = a1 - lambda a2;   then (head_norm) o <- o * rsqrt(mean(o^2) + eps);   o <- o * out_scale
// ---------------------------------------------------------------------------------------------------------------------------------
constexpr int kAttnThreads = 128;
constexpr int kAttnKT = 128;
constexpr int kAttnMaxV = 4;  // value dims per thread: Dv <= 512

template <typename ST, int MAPS>
__global__ void __launch_bounds__(kAttnThreads) paged_multimap_attention_kernel(
    ST* __restrict__ out, long long out_stride, const ST* __restrict__ q, long long q_stride, const ST* __restrict__ kpool,
    const ST* __restrict__ vpool, const int* __restrict__ tok_slot, const int* __restrict__ tok_pos, const int* __restrict__ block_table,
    int max_blocks, int H, int G, int D, int Dv, float scale, float lambda, float out_scale, float eps, int head_norm, int page, int chunk,
    int window, const float* __restrict__ sinks, AttnExtra ex) {
  extern __shared__ float sm[];
  float* qs = sm;                      // [MAPS * D]
  float* ps = qs + MAPS * D;           // [MAPS][KT]
  float* red = ps + MAPS * kAttnKT;    // [33]
  __shared__ int pages[kAttnKT];       // page of every key of the tile (KT keys span at most KT pages)

  const int t = blockIdx.x, h = blockIdx.y, g = h / (H / G);
  const int pos = tok_pos[t], slot = tok_slot[t];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int* bt = block_table + (size_t)slot * max_blocks;

  const ST* qrow = q + (size_t)t * q_stride + (size_t)h * MAPS * D;
  for (int i = threadIdx.x; i < MAPS * D; i += blockDim.x) qs[i] = ldf(qrow + i);

  float m_run[MAPS], l_run[MAPS], acc[MAPS][kAttnMaxV];
#pragma unroll
  for (int m = 0; m < MAPS; ++m) {
    // a sink is one more term exp(sink) of the denominator that carries no value: the running maximum and sum start from it
    m_run[m] = sinks != nullptr ? sinks[h] : -INFINITY;
    l_run[m] = sinks != nullptr ? 1.f : 0.f;
#pragma unroll
    for (int j = 0; j < kAttnMaxV; ++j) acc[m][j] = 0.f;
  }
  const int n_keys = pos + 1;
  const int first = first_key(pos, chunk, window), kept = min(ex.keep_first, first);
  const float slope = ex.slopes != nullptr ? ex.slopes[h] : 0.f;
  // two runs of keys: the kept first positions that lie before the window, then the window (or chunk, or everything) up to the token itself
  for (int seg = kept > 0 ? 0 : 1; seg < 2; ++seg)
  for (int base = seg == 0 ? 0 : first, hi = seg == 0 ? kept : n_keys; base < hi; base += kAttnKT) {
    const int nk = min(kAttnKT, hi - base);
    __syncthreads();  // previous tile's ps / pages fully consumed (and qs written, first time)
    for (int j = threadIdx.x; j < nk; j += blockDim.x) pages[j] = bt[(base + j) / page];
    __syncthreads();
    // scores: warp per key
    for (int j = warp; j < nk; j += kAttnThreads / 32) {
      const int kj = base + j;
      const ST* kr = kpool + (((size_t)pages[j] * page + (kj % page)) * G + g) * (size_t)(MAPS * D);
#pragma unroll
      for (int m = 0; m < MAPS; ++m) {
        float d = 0.f;
        for (int i = lane; i < D; i += 32) d += qs[m * D + i] * ldf(kr + m * D + i);
        d = warp_sum(d);
        if (lane == 0) ps[m * kAttnKT + j] = d * scale - slope * (float)(pos - kj);
      }
    }
    __syncthreads();
    // online softmax per map
    float corr[MAPS];
#pragma unroll
    for (int m = 0; m < MAPS; ++m) {
      float mx = -INFINITY;
      for (int j = threadIdx.x; j < nk; j += blockDim.x) mx = fmaxf(mx, ps[m * kAttnKT + j]);
      mx = block_max(mx, red);
      const float m_new = fmaxf(m_run[m], mx);
      float s = 0.f;
      for (int j = threadIdx.x; j < nk; j += blockDim.x) {
        const float p = expf(ps[m * kAttnKT + j] - m_new);
        ps[m * kAttnKT + j] = p;
        s += p;
      }
      s = block_sum(s, red);
      corr[m] = expf(m_run[m] - m_new);  // 0 on the first tile (m_run = -inf)
      l_run[m] = l_run[m] * corr[m] + s;
      m_run[m] = m_new;
    }
    __syncthreads();
    // weighted values: thread owns output dims
#pragma unroll
    for (int j = 0; j < kAttnMaxV; ++j) {
      const int d = threadIdx.x + j * kAttnThreads;
      if (d < Dv) {
        float a[MAPS];
#pragma unroll
        for (int m = 0; m < MAPS; ++m) a[m] = acc[m][j] * corr[m];
        for (int kk = 0; kk < nk; ++kk) {
          const int kj = base + kk;
          const float v = ldf(vpool + (((size_t)pages[kk] * page + (kj % page)) * G + g) * (size_t)Dv + d);
#pragma unroll
          for (int m = 0; m < MAPS; ++m) a[m] += ps[m * kAttnKT + kk] * v;
        }
#pragma unroll
        for (int m = 0; m < MAPS; ++m) acc[m][j] = a[m];
      }
    }
  }
  // epilogue
  float o[kAttnMaxV];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kAttnMaxV; ++j) {
    const int d = threadIdx.x + j * kAttnThreads;
    o[j] = 0.f;
    if (d < Dv) {
      float v = acc[0][j] / l_run[0];
      if (MAPS == 2) v -= lambda * (acc[MAPS - 1][j] / l_run[MAPS - 1]);
      o[j] = v;
      ss += v * v;
    }
  }
  float r = out_scale;
  if (head_norm) {
    ss = block_sum(ss, red);
    r *= 1.f / sqrtf(ss / (float)Dv + eps);
  }
  if (ex.gate != nullptr) r *= sigmoid_f(ldf(static_cast<const ST*>(ex.gate) + (size_t)t * ex.gate_stride + h));
  ST* orow = out + (size_t)t * out_stride + (size_t)h * Dv;
#pragma unroll
  for (int j = 0; j < kAttnMaxV; ++j) {
    const int d = threadIdx.x + j * kAttnThreads;
    if (d < Dv) stf(orow + d, o[j] * r);
  }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// Prompt portions on the tensor cores (bfloat16 storage).  One block = 64 consecutive query rows of one entry x one (head, map); keys are
// walked in tiles of KT (32 or 64) positions through the block table.  S = Q K^T with mma.sync m16n8k16 (bf16 operands are exact, fp32 accumulation: the
// scores are fp32), online softmax in fp32 registers, and P V with the fp32 weights split into PSPLIT bfloat16 terms (p = hi + mid + lo, 24
// mantissa bits) so that the weights enter the product at fp32 precision although the tensor cores take 16-bit operands.  The normalised
// per-map outputs go to an fp32 scratch [token][head][map][Dv]; multimap_combine_kernel finishes the head.
// ---------------------------------------------------------------------------------------------------------------------------------
constexpr int kTileQ = 64, kTileK = 64, kPad = 8;

template <int NVT, int PSPLIT, int KT>  // NVT = Dv / 16, KT keys per tile (64, or 32: less shared memory and fewer registers, 3 blocks per SM)
__global__ void __launch_bounds__(128, KT == 32 ? 3 : 2) tile_attention_kernel(
    float* __restrict__ a_out, const __nv_bfloat16* __restrict__ q, long long q_stride, const __nv_bfloat16* __restrict__ kpool,
    const __nv_bfloat16* __restrict__ vpool, const int* __restrict__ tile_entry, const int* __restrict__ tile_row0,
    const int* __restrict__ entry_start, const int* __restrict__ entry_len, const int* __restrict__ entry_slot, const int* __restrict__ entry_pos0,
    const int* __restrict__ block_table, int max_blocks, int H, int G, int maps, int D, float scale, int page, int chunk, int window,
    const float* __restrict__ sinks, int keep, const float* __restrict__ slopes) {
  extern __shared__ __align__(16) unsigned char smraw[];
  constexpr int Dv = NVT * 16;
  const int SD = D + kPad, SV = Dv + kPad;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw);
  __nv_bfloat16* Ks = Qs + kTileQ * SD;
  __nv_bfloat16* Vs = Ks + 2 * KT * SD;  // two key buffers, then two value buffers
  const int tile = blockIdx.x, hm = blockIdx.y, h = hm / maps, m = hm - h * maps, g = h / (H / G);
  const int e = tile_entry[tile], r0 = tile_row0[tile];
  const int n_rows = min(kTileQ, entry_len[e] - r0);
  const int tok0 = entry_start[e] + r0, qpos0 = entry_pos0[e] + r0;
  const int* bt = block_table + (size_t)entry_slot[e] * max_blocks;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int dch = D >> 3;  // 16-byte chunks per q / k row
  for (int c = tid; c < kTileQ * dch; c += 128) {
    const int r = c / dch, cc = c - r * dch;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < n_rows) v = *reinterpret_cast<const uint4*>(q + (size_t)(tok0 + r) * q_stride + (size_t)(h * maps + m) * D + cc * 8);
    *reinterpret_cast<uint4*>(Qs + r * SD + cc * 8) = v;
  }
  float o[2 * NVT][4];
#pragma unroll
  for (int i = 0; i < 2 * NVT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const int last_qpos = qpos0 + n_rows - 1;
  const int n_kt = last_qpos / KT + 1;
  const int kt_lo = first_key(qpos0, chunk, window) / KT;  // the tile's first row sees furthest back
  const int n_pre = kept_tiles(first_key(qpos0, chunk, window), keep, KT), n_walk = n_pre + n_kt - kt_lo;  // kept first positions, then the rest
  auto tile_at = [&](int i) { return i < n_pre ? i : kt_lo + i - n_pre; };
  const float slope2 = slopes != nullptr ? slopes[h] * 1.4426950408889634f : 0.f;
  const float scale_log2 = scale * 1.4426950408889634f;
  const int qrow = warp * 16 + (lane >> 2);  // this thread's rows: qrow, qrow + 8
  const int fk[2] = {first_key(qpos0 + qrow, chunk, window), first_key(qpos0 + qrow + 8, chunk, window)};
  const int warp_fk = first_key(min(last_qpos, qpos0 + warp * 16 + 15), chunk, window);  // the largest first key among the warp's rows
  // a sink is one more term of the denominator without a value: the running maximum starts from it and one lane of the row's quad carries its 1
  const float sink2 = sinks != nullptr ? sinks[h] * 1.4426950408889634f : -INFINITY;
  const float l0 = sinks != nullptr && (lane & 3) == 0 ? 1.f : 0.f;
  float m_run[2] = {sink2, sink2}, l_run[2] = {l0, l0};
  // key / value tiles are double-buffered: tile kt + 1 streams in with cp.async while tile kt is multiplied
  constexpr int TPR = 128 / KT;
  // TPR threads per key row, alternating 16-byte chunks: one block-table lookup per thread and tile, made one tile ahead of its use so
  // that the lookup's latency hides behind a tile of arithmetic
  auto cell_of = [&](int kt) -> long long {
    const int kp = kt * KT + tid / TPR;
    return kp <= last_qpos ? (long long)bt[kp / page] * page + kp % page : -1;
  };
  auto load_kv = [&](int kt, int buf, long long cell) {
    const int r = tid / TPR;
    __nv_bfloat16* Kd = Ks + (size_t)buf * KT * SD + r * SD;
    __nv_bfloat16* Vd = Vs + (size_t)buf * KT * SV + r * SV;
    if (cell >= 0) {
      const __nv_bfloat16* ksrc = kpool + ((cell * G + g) * maps + m) * (size_t)D;
      const __nv_bfloat16* vsrc = vpool + (cell * G + g) * (size_t)Dv;
      for (int cc = tid % TPR; cc < dch; cc += TPR) cp_async16(Kd + cc * 8, ksrc + cc * 8);
#pragma unroll
      for (int cc = tid % TPR; cc < Dv / 8; cc += TPR) cp_async16(Vd + cc * 8, vsrc + cc * 8);
    } else {
      for (int cc = tid % TPR; cc < dch; cc += TPR) *reinterpret_cast<uint4*>(Kd + cc * 8) = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int cc = tid % TPR; cc < Dv / 8; cc += TPR) *reinterpret_cast<uint4*>(Vd + cc * 8) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  load_kv(tile_at(0), 0, cell_of(tile_at(0)));
  long long cell_next = 1 < n_walk ? cell_of(tile_at(1)) : -1;
  for (int wi = 0; wi < n_walk; ++wi) {
    const int kt = tile_at(wi);
    if (wi + 1 < n_walk) {
      load_kv(tile_at(wi + 1), (wi + 1) & 1, cell_next);
      if (wi + 2 < n_walk) cell_next = cell_of(tile_at(wi + 2));
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const __nv_bfloat16* Kc = Ks + (size_t)(wi & 1) * KT * SD;
    const __nv_bfloat16* Vc = Vs + (size_t)(wi & 1) * KT * SV;
    float s[KT / 8][4];
#pragma unroll
    for (int i = 0; i < KT / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    for (int ks = 0; ks < D; ks += 16) {
      uint32_t a[4];
      ldsm_x4(a, Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * SD + ks + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < KT / 16; ++np) {
        uint32_t b[4];
        ldsm_x4(b, Kc + (np * 16 + (lane & 7) + (lane >> 4) * 8) * SD + ks + ((lane >> 3) & 1) * 8);
        mma_bf16(s[2 * np], a, b[0], b[1]);
        mma_bf16(s[2 * np + 1], a, b[2], b[3]);
      }
    }
    // scale, causal mask, online softmax (rows qrow and qrow + 8; a row's columns live in the 4 lanes of a quad)
    float mx[2] = {-INFINITY, -INFINITY};
    const bool diagonal = kt * KT + KT - 1 > qpos0 + warp * 16 || kt * KT < warp_fk;
    const bool biased = slope2 != 0.f;
#pragma unroll
    for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v = s[nt][j] * scale_log2;
        if (diagonal || biased) {  // warp-uniform: only tiles that reach past this warp's first row, or start before a row's first key, need a mask
          const int kpos = kt * KT + nt * 8 + (lane & 3) * 2 + (j & 1);
          const int qp = qpos0 + qrow + (j >> 1) * 8;
          if (biased) v -= slope2 * (float)(qp - kpos);
          if (diagonal && !key_visible(kpos, qp, fk[j >> 1], keep)) v = -INFINITY;
        }
        s[nt][j] = v;
        mx[j >> 1] = fmaxf(mx[j >> 1], v);
      }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      corr[r] = m_new == -INFINITY ? 1.f : fast_exp2(m_run[r] - m_new);
      m_run[r] = m_new;
      l_run[r] *= corr[r];
    }
#pragma unroll
    for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float mm = m_run[j >> 1];
        const float p = mm == -INFINITY ? 0.f : fast_exp2(s[nt][j] - mm);
        s[nt][j] = p;
        l_run[j >> 1] += p;
      }
#pragma unroll
    for (int i = 0; i < 2 * NVT; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
    // P V: value fragments of NVG column blocks are held while the PSPLIT terms of the weights pass, so that two products into the same
    // accumulator are 2 NVG instructions apart
    constexpr int NVG = NVT % 4 == 0 ? 4 : 2;
#pragma unroll
    for (int kk = 0; kk < KT / 16; ++kk) {  // 16 keys per step
      uint32_t a[PSPLIT][4];
#pragma unroll
      for (int part = 0; part < 4; ++part) {
        const int nt = 2 * kk + (part >> 1), j0 = (part & 1) * 2;
        float r0v = s[nt][j0], r1v = s[nt][j0 + 1];
#pragma unroll
        for (int sp = 0; sp < PSPLIT; ++sp) a[sp][part] = split_bf16x2(r0v, r1v);
      }
#pragma unroll
      for (int nv0 = 0; nv0 < NVT; nv0 += NVG) {
        uint32_t b[NVG][4];
#pragma unroll
        for (int i = 0; i < NVG; ++i)
          ldsm_x4_trans(b[i], Vc + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * SV + (nv0 + i) * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int sp = 0; sp < PSPLIT; ++sp)
#pragma unroll
          for (int i = 0; i < NVG; ++i) {
            mma_bf16(o[2 * (nv0 + i)], a[sp], b[i][0], b[i][1]);
            mma_bf16(o[2 * (nv0 + i) + 1], a[sp], b[i][2], b[i][3]);
          }
      }
    }
    __syncthreads();  // every warp is done with this buffer before tile kt + 2 streams into it
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = qrow + r * 8;
    if (row < n_rows) {
      const float inv = 1.f / l_run[r];
      float* dst = a_out + (((size_t)(tok0 + row) * H + h) * maps + m) * (size_t)Dv + (lane & 3) * 2;
#pragma unroll
      for (int i = 0; i < 2 * NVT; ++i) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
    }
  }
}

// finish a head from its per-map outputs: o = a1 [- lambda a2]; (head_norm) unit RMS; times out_scale.  One warp per (listed token, head).
template <typename ST>
__global__ void multimap_combine_kernel(ST* __restrict__ out, long long out_stride, const float* __restrict__ a_in, const int* __restrict__ tok_list,
                                        int n_list, int H, int maps, int Dv, float lambda, float out_scale, float eps, int head_norm,
                                        const ST* __restrict__ gate, long long gate_stride) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= n_list * H) return;
  const int t = tok_list[w / H], h = w % H;
  const float* a = a_in + ((size_t)t * H + h) * maps * (size_t)Dv;
  float ss = 0.f;
  for (int i = lane; i < Dv; i += 32) {
    const float v = maps == 2 ? a[i] - lambda * a[Dv + i] : a[i];
    ss += v * v;
  }
  ss = warp_sum(ss);
  float r = head_norm ? out_scale / sqrtf(ss / (float)Dv + eps) : out_scale;
  if (gate != nullptr) r *= sigmoid_f(ldf(gate + (size_t)t * gate_stride + h));
  ST* dst = out + (size_t)t * out_stride + (size_t)h * Dv;
  for (int i = lane; i < Dv; i += 32) stf(dst + i, (maps == 2 ? a[i] - lambda * a[Dv + i] : a[i]) * r);
}

// ---------------------------------------------------------------------------------------------------------------------------------
// Single tokens on the tensor cores (bfloat16 storage).  The R = H / G query heads that share a key/value head are the rows of one m16n8k16
// tile, so a key row is loaded once for the group and scored by the tensor cores instead of R warp reductions.  One block = (listed token,
// kv head, map, share of the keys); its four warps each take 16 of the 64 keys of a tile that the block stages with cp.async (double
// buffered), keep their own running maximum / sum / accumulators, and merge through shared memory at the end.  The block writes
// [maximum (base-2 domain), sum, unnormalised output] per head to part[listed token][head][map][share]; group_merge_kernel merges the
// shares, combines the maps and finishes the head.
// ---------------------------------------------------------------------------------------------------------------------------------
template <int NVT, int PSPLIT>
__global__ void __launch_bounds__(128) group_attention_kernel(
    float* __restrict__ part, const __nv_bfloat16* __restrict__ q, long long q_stride, const __nv_bfloat16* __restrict__ kpool,
    const __nv_bfloat16* __restrict__ vpool, const int* __restrict__ tok_list, const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
    const int* __restrict__ block_table, int max_blocks, int H, int G, int maps, int D, float scale, int page, int shares, int chunk, int window,
    int keep, const float* __restrict__ slopes) {
  extern __shared__ __align__(16) unsigned char smraw[];
  constexpr int Dv = NVT * 16;
  const int SD = D + kPad, SV = Dv + kPad, R = H / G;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw);  // 16 rows, the group's heads first
  __nv_bfloat16* Ks = Qs + 16 * SD;
  __nv_bfloat16* Vs = Ks + 2 * kTileK * SD;
  const int li = blockIdx.x, g = blockIdx.y / maps, m = blockIdx.y - g * maps, share = blockIdx.z;
  const int t = tok_list[li], pos = tok_pos[t];
  const int* bt = block_table + (size_t)tok_slot[t] * max_blocks;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int dch = D >> 3;
  const int first = first_key(pos, chunk, window), kt_lo = first / kTileK;
  // the walk over tiles (kept first positions, then from the first visible key on) is shared out: walk indices [kt0, kt1) are this block's
  const int n_pre = kept_tiles(first, keep, kTileK), n_walk = n_pre + pos / kTileK + 1 - kt_lo, per = (n_walk + shares - 1) / shares;
  const int kt0 = share * per, kt1 = min(n_walk, kt0 + per);
  auto tile_at = [&](int i) { return i < n_pre ? i : kt_lo + i - n_pre; };
  float* pout = part + ((((size_t)li * H + g * R) * maps + m) * shares + share) * (size_t)(2 + Dv);  // head g R + r: + r maps shares (2 + Dv)
  const size_t head_step = (size_t)maps * shares * (2 + Dv);
  if (kt0 >= kt1) {  // a share without keys weighs nothing in the merge
    for (int r = tid; r < R; r += 128) { pout[r * head_step] = -INFINITY; pout[r * head_step + 1] = 0.f; }
    return;
  }
  for (int c = tid; c < 16 * dch; c += 128) {
    const int r = c / dch, cc = c - r * dch;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < R) v = *reinterpret_cast<const uint4*>(q + (size_t)t * q_stride + (size_t)((g * R + r) * maps + m) * D + cc * 8);
    *reinterpret_cast<uint4*>(Qs + r * SD + cc * 8) = v;
  }
  float o[2 * NVT][4];
#pragma unroll
  for (int i = 0; i < 2 * NVT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float scale_log2 = scale * 1.4426950408889634f;
  // two threads per key row, alternating 16-byte chunks: one block-table lookup per thread and tile, made one tile ahead of its use so
  // that the lookup's latency hides behind a tile of arithmetic
  auto cell_of = [&](int kt) -> long long {
    const int kp = kt * kTileK + (tid >> 1);
    return kp <= pos ? (long long)bt[kp / page] * page + kp % page : -1;
  };
  auto load_kv = [&](int kt, int buf, long long cell) {
    const int r = tid >> 1;
    __nv_bfloat16* Kd = Ks + (size_t)buf * kTileK * SD + r * SD;
    __nv_bfloat16* Vd = Vs + (size_t)buf * kTileK * SV + r * SV;
    if (cell >= 0) {
      const __nv_bfloat16* ksrc = kpool + ((cell * G + g) * maps + m) * (size_t)D;
      const __nv_bfloat16* vsrc = vpool + (cell * G + g) * (size_t)Dv;
      for (int cc = tid & 1; cc < dch; cc += 2) cp_async16(Kd + cc * 8, ksrc + cc * 8);
#pragma unroll
      for (int cc = tid & 1; cc < Dv / 8; cc += 2) cp_async16(Vd + cc * 8, vsrc + cc * 8);
    } else {
      for (int cc = tid & 1; cc < dch; cc += 2) *reinterpret_cast<uint4*>(Kd + cc * 8) = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int cc = tid & 1; cc < Dv / 8; cc += 2) *reinterpret_cast<uint4*>(Vd + cc * 8) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  load_kv(tile_at(kt0), 0, cell_of(tile_at(kt0)));
  long long cell_next = kt0 + 1 < kt1 ? cell_of(tile_at(kt0 + 1)) : -1;
  float slope2[2] = {0.f, 0.f};  // of this thread's rows (heads g R + row, g R + row + 8)
  if (slopes != nullptr) {
#pragma unroll
    for (int r = 0; r < 2; ++r)
      if ((lane >> 2) + r * 8 < R) slope2[r] = slopes[g * R + (lane >> 2) + r * 8] * 1.4426950408889634f;
  }
  for (int wi = kt0; wi < kt1; ++wi) {
    const int buf = (wi - kt0) & 1, kt = tile_at(wi);
    if (wi + 1 < kt1) {
      load_kv(tile_at(wi + 1), buf ^ 1, cell_next);
      if (wi + 2 < kt1) cell_next = cell_of(tile_at(wi + 2));
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const __nv_bfloat16* Kc = Ks + (size_t)buf * kTileK * SD;
    const __nv_bfloat16* Vc = Vs + (size_t)buf * kTileK * SV;
    float s[2][4];  // this warp's 16 keys of the tile: two blocks of 8
#pragma unroll
    for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    for (int ks = 0; ks < D; ks += 16) {
      uint32_t a[4], b[4];
      ldsm_x4(a, Qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * SD + ks + (lane >> 4) * 8);
      ldsm_x4(b, Kc + (warp * 16 + (lane & 7) + (lane >> 4) * 8) * SD + ks + ((lane >> 3) & 1) * 8);
      mma_bf16(s[0], a, b[0], b[1]);
      mma_bf16(s[1], a, b[2], b[3]);
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kpos = kt * kTileK + warp * 16 + nt * 8 + (lane & 3) * 2 + (j & 1);
        const float v = key_visible(kpos, pos, first, keep) ? s[nt][j] * scale_log2 - slope2[j >> 1] * (float)(pos - kpos) : -INFINITY;
        s[nt][j] = v;
        mx[j >> 1] = fmaxf(mx[j >> 1], v);
      }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      corr[r] = m_new == -INFINITY ? 1.f : fast_exp2(m_run[r] - m_new);
      m_run[r] = m_new;
      l_run[r] *= corr[r];
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float mm = m_run[j >> 1];
        const float p = mm == -INFINITY ? 0.f : fast_exp2(s[nt][j] - mm);
        s[nt][j] = p;
        l_run[j >> 1] += p;
      }
#pragma unroll
    for (int i = 0; i < 2 * NVT; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
    uint32_t a[PSPLIT][4];
#pragma unroll
    for (int pt = 0; pt < 4; ++pt) {
      float r0v = s[pt >> 1][(pt & 1) * 2], r1v = s[pt >> 1][(pt & 1) * 2 + 1];
#pragma unroll
      for (int sp = 0; sp < PSPLIT; ++sp) a[sp][pt] = split_bf16x2(r0v, r1v);
    }
    constexpr int NVG = NVT % 4 == 0 ? 4 : 2;
#pragma unroll
    for (int nv0 = 0; nv0 < NVT; nv0 += NVG) {
      uint32_t b[NVG][4];
#pragma unroll
      for (int i = 0; i < NVG; ++i)
        ldsm_x4_trans(b[i], Vc + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * SV + (nv0 + i) * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int sp = 0; sp < PSPLIT; ++sp)
#pragma unroll
        for (int i = 0; i < NVG; ++i) {
          mma_bf16(o[2 * (nv0 + i)], a[sp], b[i][0], b[i][1]);
          mma_bf16(o[2 * (nv0 + i) + 1], a[sp], b[i][2], b[i][3]);
        }
    }
    __syncthreads();
  }
  // merge the four warps: [warp][row][2 + Dv] floats over the key and value buffers (all tiles are consumed; 4 R (2 + Dv) floats fit for R <= 16)
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  float* mg = reinterpret_cast<float*>(Ks);
  const int row = lane >> 2;  // rows 8 .. 15 hold no head when R <= 8
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int rr = row + r * 8;
    if (rr < R) {
      float* w = mg + ((size_t)warp * R + rr) * (2 + Dv);
      if ((lane & 3) == 0) { w[0] = m_run[r]; w[1] = l_run[r]; }
#pragma unroll
      for (int i = 0; i < 2 * NVT; ++i) {
        w[2 + i * 8 + (lane & 3) * 2] = o[i][2 * r];
        w[2 + i * 8 + (lane & 3) * 2 + 1] = o[i][2 * r + 1];
      }
    }
  }
  __syncthreads();
  for (int c = tid; c < R * (Dv + 1); c += 128) {
    const int r = c / (Dv + 1), d = c - r * (Dv + 1);  // d == Dv: the sum
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, mg[((size_t)w * R + r) * (2 + Dv)]);
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float* src = mg + ((size_t)w * R + r) * (2 + Dv);
      const float f = src[0] == -INFINITY ? 0.f : fast_exp2(src[0] - M);
      acc += f * (d == Dv ? src[1] : src[2 + d]);
    }
    if (d == Dv) { pout[r * head_step] = M; pout[r * head_step + 1] = acc; }
    else pout[r * head_step + 2 + d] = acc;
  }
}

// merge the shares of every (listed token, head, map), then finish the head as multimap_combine_kernel does.  One warp per (token, head).
template <typename ST>
__global__ void group_merge_kernel(ST* __restrict__ out, long long out_stride, const float* __restrict__ part, const int* __restrict__ tok_list,
                                   int n_list, int H, int maps, int Dv, int shares, float lambda, float out_scale, float eps, int head_norm,
                                   const float* __restrict__ sinks, const ST* __restrict__ gate, long long gate_stride) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= n_list * H) return;
  const int li = w / H, h = w - li * H, t = tok_list[li];
  const float* base = part + ((size_t)li * H + h) * maps * shares * (size_t)(2 + Dv);
  float ov[8];  // Dv <= 256
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ov[j] = 0.f;
  for (int mm = 0; mm < maps; ++mm) {
    const float* pm = base + (size_t)mm * shares * (2 + Dv);
    const float sink2 = sinks != nullptr ? sinks[h] * 1.4426950408889634f : -INFINITY;  // the sink: a share of maximum sink, sum 1, no output
    float M = sink2;
    for (int z = 0; z < shares; ++z) M = fmaxf(M, pm[(size_t)z * (2 + Dv)]);
    float den = sinks != nullptr ? fast_exp2(sink2 - M) : 0.f, num[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) num[j] = 0.f;
    for (int z = 0; z < shares; ++z) {
      const float* src = pm + (size_t)z * (2 + Dv);
      if (src[0] == -INFINITY) continue;  // a share without keys wrote no output
      const float f = fast_exp2(src[0] - M);
      den += f * src[1];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (lane + 32 * j < Dv) num[j] += f * src[2 + lane + 32 * j];
    }
    const float wgt = (mm == 0 ? 1.f : -lambda) / den;  // maps beyond the first enter with -lambda (two maps: a1 - lambda a2)
#pragma unroll
    for (int j = 0; j < 8; ++j) ov[j] += wgt * num[j];
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) ss += ov[j] * ov[j];
  ss = warp_sum(ss);
  float r = head_norm ? out_scale / sqrtf(ss / (float)Dv + eps) : out_scale;
  if (gate != nullptr) r *= sigmoid_f(ldf(gate + (size_t)t * gate_stride + h));
  ST* dst = out + (size_t)t * out_stride + (size_t)h * Dv;
#pragma unroll
  for (int j = 0; j < 8; ++j)
    if (lane + 32 * j < Dv) stf(dst + lane + 32 * j, ov[j] * r);
}

// ---------------------------------------------------------------------------------------------------------------------------------
// gated delta rule, step 1: per token, short causal convolution + silu over the q | k | v channels (taps before the portion come from
// the sequence's convolution state, taps before the sequence's start are zero), unit-length q (times D^-1/2) and k per head, the write
// strength beta = sigmoid(b) and the decay exp(-exp(A_log) softplus(a + dt_bias)) per head.  All fp32 from the projections on.
//   projection row: [G*D q | G*D k | H*Dv v | H*Dv output gate | H b | H a]
//   prepared row (fp32): [G*D q | G*D k | H*Dv v | H beta | H decay]
//   convolution state (fp32): [slots][taps - 1][C], oldest first, C = 2 G D + H Dv
// ---------------------------------------------------------------------------------------------------------------------------------
// One block per (token, unit); the units of a token are its G q heads, its G k heads (D channels each, made unit vectors) and its H value
// heads (Dv channels): single tokens of a small batch still fill the SMs.  Unit 0 also writes the token's write strengths and decays.
constexpr int kPrepThreads = 128, kPrepPerThread = 8;  // channels of a unit <= 1024

template <typename ST>
__global__ void __launch_bounds__(kPrepThreads) delta_prepare_kernel(
    float* __restrict__ prep, const ST* __restrict__ proj, long long stride, const float* __restrict__ conv_w,
    const float* __restrict__ conv_state, const float* __restrict__ a_log, const float* __restrict__ dt_bias, const int* __restrict__ tok_entry,
    const int* __restrict__ tok_pos, const int* __restrict__ entry_start, const int* __restrict__ entry_slot, int H, int G, int D, int Dv,
    int taps, float unit_eps) {
  __shared__ float red[33];
  const int t = blockIdx.x, u = blockIdx.y;
  const int C = 2 * G * D + H * Dv;
  const int P = C + 2 * H;
  const bool qk = u < 2 * G;
  const int c0 = qk ? u * D : 2 * G * D + (u - 2 * G) * Dv, n = qk ? D : Dv;
  const int e = tok_entry[t], pos = tok_pos[t];
  const int local = t - entry_start[e];
  const float* st = conv_state + (size_t)entry_slot[e] * (taps - 1) * C;
  float y[kPrepPerThread];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < kPrepPerThread; ++k) {
    const int i = threadIdx.x + k * kPrepThreads;
    y[k] = 0.f;
    if (i < n) {
      const int c = c0 + i;
      float a = 0.f;
      for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        if (pos - back < 0) continue;
        float x;
        if (local - back >= 0) x = ldf(proj + (size_t)(t - back) * stride + c);
        else x = st[(size_t)(taps - 1 + local - back) * C + c];
        a += conv_w[(size_t)c * taps + j] * x;
      }
      y[k] = silu_f(a);
      ss += y[k] * y[k];
    }
  }
  float r = 1.f;
  if (qk) {  // block-uniform
    ss = block_sum(ss, red);
    r = 1.f / sqrtf(ss + unit_eps);
    if (u < G) r *= 1.f / sqrtf((float)D);
  }
  float* o = prep + (size_t)t * P;
#pragma unroll
  for (int k = 0; k < kPrepPerThread; ++k) {
    const int i = threadIdx.x + k * kPrepThreads;
    if (i < n) o[c0 + i] = y[k] * r;
  }
  if (u != 0) return;
  const ST* row = proj + (size_t)t * stride;
  for (int hh = threadIdx.x; hh < H; hh += kPrepThreads) {
    const float b = ldf(row + C + H * Dv + hh);
    const float a = ldf(row + C + H * Dv + H + hh) + dt_bias[hh];
    const float sp = a > 20.f ? a : log1pf(expf(a));
    o[C + hh] = 1.f / (1.f + expf(-b));
    o[C + H + hh] = expf(-expf(a_log[hh]) * sp);
  }
}

// step 1b: the sequence's convolution state after the portion = its last taps-1 inputs (older ones shift out)
template <typename ST>
__global__ void delta_conv_state_kernel(float* __restrict__ conv_state, const ST* __restrict__ proj, long long stride,
                                        const int* __restrict__ entry_start, const int* __restrict__ entry_len, const int* __restrict__ entry_slot,
                                        const int* __restrict__ entry_pos0, int C, int taps) {
  const int e = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int n = entry_len[e], s0 = entry_start[e], keep = taps - 1;
  float* st = conv_state + (size_t)entry_slot[e] * keep * C;
  const bool fresh = entry_pos0[e] == 0;
  float tmp[16];
  for (int i = 0; i < keep; ++i) {
    const int src = n - keep + i;  // index in the portion, negative: older than the portion
    if (src >= 0) tmp[i] = ldf(proj + (size_t)(s0 + src) * stride + c);
    else tmp[i] = fresh ? 0.f : st[(size_t)(keep + src) * C + c];
  }
  for (int i = 0; i < keep; ++i) st[(size_t)i * C + c] = tmp[i];
}

// step 2: the recurrence.  Columns of a head's [D, Dv] state are independent, so a block owns 128 / PARTS columns of one (entry, head):
// thread (column, part) keeps rows [part Q, (part + 1) Q) of its column in registers (Q = DP / PARTS, D <= DP); the parts of a column sit in
// adjacent lanes and meet through shuffles.  With PARTS = 1 every lane of a warp reads the same q / k words from shared memory (a
// broadcast).  Tokens are staged CH at a time (q | k | v of the block's columns | beta | decay) with cp.async into a double buffer, so that no
// global load sits on the token-to-token dependency chain.  Per token, in this order:
//   S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
template <int PARTS>
__device__ __forceinline__ float part_sum(float v) {
#pragma unroll
  for (int o = 1; o < PARTS; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int DP, int PARTS, int CH, int CPT, bool VEC>  // VEC: rows of `prep`, D and Dv are multiples of 4 floats: stage with 16-byte copies
__global__ void __launch_bounds__(128) delta_scan_kernel(float* __restrict__ o_raw, const float* __restrict__ prep, float* __restrict__ state,
                                                         const int* __restrict__ entry_start, const int* __restrict__ entry_len,
                                                         const int* __restrict__ entry_slot, const int* __restrict__ entry_pos0, int H, int G, int D,
                                                         int Dv) {
  extern __shared__ __align__(16) float sm[];  // [2][CH][ROW]
  constexpr int Q = DP / PARTS, SEG = Q + 4, TC = 128 / PARTS, COLS = TC * CPT;  // a part's q / k segment is padded by 16 bytes: parts hit different banks
  constexpr int QK = PARTS * SEG, ROW = 2 * QK + COLS + 4;
  const int e = blockIdx.x, h = blockIdx.y, cg = blockIdx.z, g = h / (H / G);
  const int tid = threadIdx.x, part = tid % PARTS, cl = tid / PARTS, col0 = cg * COLS + cl * CPT;  // CPT adjacent columns per thread
  const int C = 2 * G * D + H * Dv, P = C + 2 * H;
  const int n = entry_len[e], s0 = entry_start[e];
  const bool fresh = entry_pos0[e] == 0;
  float* Sg = state + ((size_t)entry_slot[e] * H + h) * (size_t)D * Dv;
  float S[CPT][Q];
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int j = 0; j < Q; ++j) {
      const int i = part * Q + j;
      S[c][j] = (col0 + c < Dv && !fresh && i < D) ? Sg[(size_t)i * Dv + col0 + c] : 0.f;
    }
  auto stage = [&](int chunk, int buf) {
    if (VEC) {
      constexpr int QV = Q / 4, NQK = 2 * PARTS * QV, NV = COLS / 4, ITEMS = NQK + NV + 2;
      for (int idx = tid; idx < CH * ITEMS; idx += 128) {
        const int tk = idx / ITEMS, j = idx - tk * ITEMS, t = chunk * CH + tk;
        float* base = sm + (size_t)(buf * CH + tk) * ROW;
        const float* row = prep + (size_t)(s0 + min(t, n - 1)) * P;
        float* dst;
        const float* src = nullptr;
        int bytes = 16;
        if (j < NQK) {
          const int which = j / (PARTS * QV), rem = j - which * (PARTS * QV), pp = rem / QV, w4 = rem - pp * QV, i = pp * Q + w4 * 4;
          dst = base + which * QK + pp * SEG + w4 * 4;
          if (i < D) src = row + (size_t)(which * G + g) * D + i;
        } else if (j < NQK + NV) {
          const int c4 = (j - NQK) * 4, c = cg * COLS + c4;
          dst = base + 2 * QK + c4;
          if (c < Dv) src = row + 2 * G * D + (size_t)h * Dv + c;
        } else {
          const int w = j - NQK - NV;  // beta, decay
          dst = base + 2 * QK + COLS + w;
          src = row + C + w * H + h;
          bytes = 4;
        }
        if (t >= n) src = nullptr;
        if (src != nullptr) {
          if (bytes == 16) cp_async16(dst, src); else cp_async4(dst, src);
        } else if (bytes == 16) {
          *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
          *dst = 0.f;
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      return;
    }
    for (int idx = tid; idx < CH * ROW; idx += 128) {
      const int tk = idx / ROW, j = idx - tk * ROW, t = chunk * CH + tk;
      float* dst = sm + (size_t)(buf * CH + tk) * ROW + j;
      const float* src = nullptr;
      if (t < n) {
        const float* row = prep + (size_t)(s0 + t) * P;
        if (j < 2 * QK) {
          const int which = j / QK, jj = j - which * QK, pp = jj / SEG, w = jj - pp * SEG, i = pp * Q + w;  // q (which = 0) or k row i
          if (w < Q && i < D) src = row + (size_t)(which * G + g) * D + i;
        } else if (j < 2 * QK + COLS) {
          const int c = cg * COLS + j - 2 * QK;
          if (c < Dv) src = row + 2 * G * D + (size_t)h * Dv + c;
        } else if (j == 2 * QK + COLS) {
          src = row + C + h;
        } else if (j == 2 * QK + COLS + 1) {
          src = row + C + H + h;
        }
      }
      if (src != nullptr) cp_async4(dst, src);
      else *dst = 0.f;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int n_chunks = (n + CH - 1) / CH;
  stage(0, 0);
  for (int ch = 0; ch < n_chunks; ++ch) {
    if (ch + 1 < n_chunks) {
      stage(ch + 1, (ch + 1) & 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const int cnt = min(CH, n - ch * CH);
    for (int tk = 0; tk < cnt; ++tk) {
      const float* r = sm + (size_t)((ch & 1) * CH + tk) * ROW;
      const float4* q4 = reinterpret_cast<const float4*>(r + part * SEG);
      const float4* k4 = reinterpret_cast<const float4*>(r + QK + part * SEG);
      const float beta = r[2 * QK + COLS], decay = r[2 * QK + COLS + 1];
      // a q / k word read from shared memory serves the thread's CPT columns
      float kp[CPT][4];
#pragma unroll
      for (int c = 0; c < CPT; ++c) kp[c][0] = kp[c][1] = kp[c][2] = kp[c][3] = 0.f;
#pragma unroll
      for (int j = 0; j < Q / 4; ++j) {
        const float4 kk = k4[j];
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          kp[c][0] += S[c][4 * j] * kk.x; kp[c][1] += S[c][4 * j + 1] * kk.y; kp[c][2] += S[c][4 * j + 2] * kk.z; kp[c][3] += S[c][4 * j + 3] * kk.w;
        }
      }
      float u[CPT];
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        const float kS = part_sum<PARTS>((kp[c][0] + kp[c][1]) + (kp[c][2] + kp[c][3])) * decay;
        u[c] = beta * (r[2 * QK + cl * CPT + c] - kS);
      }
      float op[CPT][4];
#pragma unroll
      for (int c = 0; c < CPT; ++c) op[c][0] = op[c][1] = op[c][2] = op[c][3] = 0.f;
#pragma unroll
      for (int j = 0; j < Q / 4; ++j) {
        const float4 kk = k4[j], qq = q4[j];
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          S[c][4 * j] = S[c][4 * j] * decay + kk.x * u[c];         op[c][0] += S[c][4 * j] * qq.x;
          S[c][4 * j + 1] = S[c][4 * j + 1] * decay + kk.y * u[c]; op[c][1] += S[c][4 * j + 1] * qq.y;
          S[c][4 * j + 2] = S[c][4 * j + 2] * decay + kk.z * u[c]; op[c][2] += S[c][4 * j + 2] * qq.z;
          S[c][4 * j + 3] = S[c][4 * j + 3] * decay + kk.w * u[c]; op[c][3] += S[c][4 * j + 3] * qq.w;
        }
      }
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        const float o = part_sum<PARTS>((op[c][0] + op[c][1]) + (op[c][2] + op[c][3]));
        if (part == 0 && col0 + c < Dv) o_raw[(size_t)(s0 + ch * CH + tk) * H * Dv + (size_t)h * Dv + col0 + c] = o;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int j = 0; j < Q; ++j) {
      const int i = part * Q + j;
      if (col0 + c < Dv && i < D) Sg[(size_t)i * Dv + col0 + c] = S[c][j];
    }
}

// step 3: per (token, head) unit-RMS read-out times a shared per-dimension weight times silu(output gate); one warp each
template <typename ST>
__global__ void delta_gate_out_kernel(ST* __restrict__ out, long long out_stride, const float* __restrict__ o_raw, const ST* __restrict__ proj,
                                      long long stride, const float* __restrict__ norm_w, int T, int H, int G, int D, int Dv, float eps) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= T * H) return;
  const int t = w / H, h = w - t * H;
  const float* o = o_raw + (size_t)t * H * Dv + (size_t)h * Dv;
  const ST* gate = proj + (size_t)t * stride + 2 * G * D + H * Dv + (size_t)h * Dv;
  float ss = 0.f;
  for (int i = lane; i < Dv; i += 32) ss += o[i] * o[i];
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)Dv + eps);
  ST* dst = out + (size_t)t * out_stride + (size_t)h * Dv;
  for (int i = lane; i < Dv; i += 32) stf(dst + i, o[i] * r * norm_w[i] * silu_f(ldf(gate + i)));
}

inline AttnExtra attn_extra(const qs_attn_extra* e) {
  return e != nullptr ? AttnExtra{e->keep_first, e->slopes, e->gate, (long long)e->gate_stride} : AttnExtra{0, nullptr, nullptr, 0};
}

template <typename ST>
int launch_attention(void* out, long long out_stride, const void* q, long long q_stride, const void* kpool, const void* vpool, const int* tok_slot,
                     const int* tok_pos, const int* block_table, int max_blocks, int T, int H, int G, int maps, int D, int Dv, float scale,
                     float lambda, float out_scale, float eps, int head_norm, int page, int chunk, int window, const float* sinks,
                     AttnExtra ex, cudaStream_t s) {
  const size_t smem = (size_t)(maps * D + maps * kAttnKT + 33) * sizeof(float);
  dim3 grid(T, H);
  if (maps == 2) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(paged_multimap_attention_kernel<ST, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    paged_multimap_attention_kernel<ST, 2><<<grid, kAttnThreads, smem, s>>>((ST*)out, out_stride, (const ST*)q, q_stride, (const ST*)kpool,
        (const ST*)vpool, tok_slot, tok_pos, block_table, max_blocks, H, G, D, Dv, scale, lambda, out_scale, eps, head_norm, page, chunk, window, sinks, ex);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(paged_multimap_attention_kernel<ST, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    paged_multimap_attention_kernel<ST, 1><<<grid, kAttnThreads, smem, s>>>((ST*)out, out_stride, (const ST*)q, q_stride, (const ST*)kpool,
        (const ST*)vpool, tok_slot, tok_pos, block_table, max_blocks, H, G, D, Dv, scale, lambda, out_scale, eps, head_norm, page, chunk, window, sinks, ex);
  }
  return check_cuda(cudaGetLastError(), "hyb_attention");
}


bool fast_attention_supported(int dtype, int heads, int kv_heads, int maps, int dim, int vdim, long long q_stride) {
  if (dtype != QS_DTYPE_BF16 || (maps != 1 && maps != 2) || kv_heads <= 0 || heads % kv_heads != 0) return false;
  const int nvt = vdim / 16, R = heads / kv_heads;
  if (dim % 16 != 0 || vdim % 16 != 0 || !(nvt == 2 || nvt == 4 || nvt == 6 || nvt == 8 || nvt == 16)) return false;
  if (R > 16 || maps * dim > 1024 || dim > 512 || q_stride % 8 != 0) return false;
  return true;
}

// keys per prompt tile: 32 keeps a block at 52 KB and 168 registers for head sizes up to 128, so that three blocks share an SM
constexpr int kTileKeysPrompt = 32;

template <int NVT, int KT>
int launch_tiles(float* scratch, const void* q, long long q_stride, const void* kpool, const void* vpool, const int* tile_entry, const int* tile_row0,
                 int n_tiles, const int* entry_start, const int* entry_len, const int* entry_slot, const int* entry_pos0, const int* block_table,
                 int max_blocks, int H, int G, int maps, int D, float scale, int page, int chunk, int window, const float* sinks, AttnExtra ex,
                 cudaStream_t s) {
  const size_t smem = ((size_t)(kTileQ + 2 * KT) * (D + kPad) + (size_t)2 * KT * (NVT * 16 + kPad)) * sizeof(__nv_bfloat16);
  static bool attr_set[kMaxDevices] = {};
  if (smem > 48 * 1024 && !attr_set[device_ordinal()]) {
    if (int rc = check_cuda(cudaFuncSetAttribute(tile_attention_kernel<NVT, 3, KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), "tile attention smem")) return rc;
    attr_set[device_ordinal()] = true;
  }
  tile_attention_kernel<NVT, 3, KT><<<dim3(n_tiles, H * maps), 128, smem, s>>>(scratch, (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)kpool,
      (const __nv_bfloat16*)vpool, tile_entry, tile_row0, entry_start, entry_len, entry_slot, entry_pos0, block_table, max_blocks, H, G, maps, D, scale, page, chunk, window, sinks,
      ex.keep_first, ex.slopes);
  return check_cuda(cudaGetLastError(), "hyb_attention tiles");
}

// key shares per (token, kv head, map) of the single-token kernel: about four blocks per SM of a 148-SM part in flight
constexpr int kGroupTargetBlocks = 592, kGroupMaxShares = 32;
inline int group_shares(int n_tokens, int G, int maps) {
  const int per = std::max(1, n_tokens * G * maps);
  return std::max(1, std::min(kGroupMaxShares, (kGroupTargetBlocks + per - 1) / per));
}

template <int NVT>
int launch_group(void* out, long long out_stride, float* part, const void* q, long long q_stride, const void* kpool, const void* vpool,
                 const int* tok_list, int n_list, const int* tok_slot, const int* tok_pos, const int* block_table, int max_blocks, int H, int G,
                 int maps, int D, float scale, float lambda, float out_scale, float eps, int head_norm, int page, int chunk, int window,
                 const float* sinks, AttnExtra ex, cudaStream_t s) {
  const size_t smem = ((size_t)(16 + 2 * kTileK) * (D + kPad) + (size_t)2 * kTileK * (NVT * 16 + kPad)) * sizeof(__nv_bfloat16);
  static bool attr_set[kMaxDevices] = {};
  if (smem > 48 * 1024 && !attr_set[device_ordinal()]) {
    if (int rc = check_cuda(cudaFuncSetAttribute(group_attention_kernel<NVT, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), "group attention smem")) return rc;
    attr_set[device_ordinal()] = true;
  }
  const int shares = group_shares(n_list, G, maps);
  group_attention_kernel<NVT, 3><<<dim3(n_list, G * maps, shares), 128, smem, s>>>(part, (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)kpool,
      (const __nv_bfloat16*)vpool, tok_list, tok_slot, tok_pos, block_table, max_blocks, H, G, maps, D, scale, page, shares, chunk, window, ex.keep_first,
      ex.slopes);
  const int warps = n_list * H;
  group_merge_kernel<__nv_bfloat16><<<(warps + 3) / 4, 128, 0, s>>>((__nv_bfloat16*)out, out_stride, part, tok_list, n_list, H, maps, NVT * 16, shares,
                                                                     lambda, out_scale, eps, head_norm, sinks, (const __nv_bfloat16*)ex.gate,
                                                                     ex.gate_stride);
  return check_cuda(cudaGetLastError(), "hyb_attention single tokens");
}

template <typename ST>
int launch_delta(void* out, long long out_stride, float* prep, float* o_raw, const void* proj, long long stride, const float* conv_w,
                 float* conv_state, float* state, const float* a_log, const float* dt_bias, const float* norm_w, const int* tok_entry,
                 const int* tok_pos, const int* entry_start, const int* entry_len, const int* entry_slot, const int* entry_pos0, int T, int E,
                 int H, int G, int D, int Dv, int taps, float unit_eps, float eps, cudaStream_t s) {
  const int C = 2 * G * D + H * Dv;
  delta_prepare_kernel<ST><<<dim3(T, 2 * G + H), kPrepThreads, 0, s>>>(prep, (const ST*)proj, stride, conv_w, conv_state, a_log, dt_bias, tok_entry,
                                                                      tok_pos, entry_start, entry_slot, H, G, D, Dv, taps, unit_eps);
  if (taps > 1)
    delta_conv_state_kernel<ST><<<dim3((C + 127) / 128, E), 128, 0, s>>>(conv_state, (const ST*)proj, stride, entry_start, entry_len, entry_slot,
                                                                          entry_pos0, C, taps);
  // 16-byte staging needs every q / k / v run of a prepared row on a 16-byte boundary
  const bool vec = D % 4 == 0 && Dv % 4 == 0 && (C + 2 * H) % 4 == 0 && (reinterpret_cast<uintptr_t>(prep) & 15) == 0;
  // rows of a column per thread: all of them up to 64 (a warp then reads q / k as broadcasts), 64 above
#define QS_SCAN(DP, PARTS, CH, CPT)                                                                                                           \
  do {                                                                                                                                        \
    constexpr int cols = 128 / PARTS * CPT;                                                                                                   \
    const size_t sm = (size_t)2 * CH * (2 * PARTS * (DP / PARTS + 4) + cols + 4) * sizeof(float);                                             \
    dim3 grid(E, H, (Dv + cols - 1) / cols);                                                                                                  \
    auto kern = vec ? delta_scan_kernel<DP, PARTS, CH, CPT, true> : delta_scan_kernel<DP, PARTS, CH, CPT, false>;                             \
    if (sm > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);                                     \
    kern<<<grid, 128, sm, s>>>(o_raw, prep, state, entry_start, entry_len, entry_slot, entry_pos0, H, G, D, Dv);                              \
  } while (0)
  // two adjacent columns per thread where the head has the columns for it: a q / k word read from shared memory then feeds two columns
  // (the scan is bound by shared-memory bandwidth: every thread reads its rows' q and k for every token)
  if (D <= 16) QS_SCAN(16, 1, 16, 1);
  else if (D <= 32) QS_SCAN(32, 1, 16, 1);
  else if (D <= 64) { if (Dv >= 128) QS_SCAN(64, 2, 16, 2); else QS_SCAN(64, 2, 16, 1); }
  else if (D <= 128) { if (Dv >= 64) QS_SCAN(128, 8, 16, 2); else QS_SCAN(128, 4, 16, 1); }
  else QS_SCAN(256, 8, 8, 1);
#undef QS_SCAN
  const int warps = T * H;
  delta_gate_out_kernel<ST><<<(warps + 3) / 4, 128, 0, s>>>((ST*)out, out_stride, o_raw, (const ST*)proj, stride, norm_w, T, H, G, D, Dv, eps);
  return check_cuda(cudaGetLastError(), "hyb_gated_delta");
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

int qs_hyb_embed(float* out, const int32_t* tokens, const int32_t* prev, const void* table, const void* pair_table, int tokens_n, int width,
                 int buckets, int64_t mul_prev, int64_t mul_cur, float scale, int copies, int dtype, void* stream) {
  QS_REQUIRE(out && tokens && table && copies >= 1, "hyb_embed: null tensor or no copies");
  QS_REQUIRE(pair_table == nullptr || (prev != nullptr && buckets > 0), "hyb_embed: the pair table needs previous tokens and buckets > 0");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  QS_DT(dtype,
        (embed_pair_kernel<__nv_bfloat16><<<tokens_n, 128, 0, s>>>(out, tokens, prev, (const __nv_bfloat16*)table, (const __nv_bfloat16*)pair_table,
                                                                    width, buckets, mul_prev, mul_cur, scale, copies)),
        (embed_pair_kernel<float><<<tokens_n, 128, 0, s>>>(out, tokens, prev, (const float*)table, (const float*)pair_table, width, buckets,
                                                           mul_prev, mul_cur, scale, copies)));
  return check_cuda(cudaGetLastError(), "hyb_embed");
}

int qs_hyb_rms_norm(void* out1, void* out2, float* x, const void* add, const float* w1, const float* w2, float offset, float eps, int tokens_n,
                    int width, int dtype, void* stream) {
  QS_REQUIRE(out1 && x && w1 && (out2 == nullptr || w2 != nullptr), "hyb_rms_norm: null tensor");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = width >= 1024 ? 256 : 128;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (width % 4 == 0 && al16(out1) && al16(out2) && al16(x) && al16(add) && al16(w1) && al16(w2)) {
    QS_DT(dtype,
          (rms_norm2_vec_kernel<__nv_bfloat16><<<tokens_n, threads, 0, s>>>((__nv_bfloat16*)out1, (__nv_bfloat16*)out2, x, (const __nv_bfloat16*)add, w1,
                                                                             w2, offset, eps, width)),
          (rms_norm2_vec_kernel<float><<<tokens_n, threads, 0, s>>>((float*)out1, (float*)out2, x, (const float*)add, w1, w2, offset, eps, width)));
    return check_cuda(cudaGetLastError(), "hyb_rms_norm");
  }
  QS_DT(dtype,
        (rms_norm2_kernel<__nv_bfloat16><<<tokens_n, threads, 0, s>>>((__nv_bfloat16*)out1, (__nv_bfloat16*)out2, x, (const __nv_bfloat16*)add, w1, w2,
                                                                       offset, eps, width)),
        (rms_norm2_kernel<float><<<tokens_n, threads, 0, s>>>((float*)out1, (float*)out2, x, (const float*)add, w1, w2, offset, eps, width)));
  return check_cuda(cudaGetLastError(), "hyb_rms_norm");
}

int qs_hyb_residual_add(float* x, const void* y, int64_t n, int dtype, void* stream) {
  QS_REQUIRE(x && y, "hyb_residual_add: null tensor");
  if (n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  QS_DT(dtype, (residual_add_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(x, (const __nv_bfloat16*)y, (size_t)n)),
        (residual_add_kernel<float><<<blocks, 256, 0, s>>>(x, (const float*)y, (size_t)n)));
  return check_cuda(cudaGetLastError(), "hyb_residual_add");
}

int qs_hyb_gelu_tanh_mul(void* out, int64_t out_stride, const void* in, int tokens_n, int ff, int dtype, void* stream) {
  QS_REQUIRE(out && in, "hyb_gelu_tanh_mul: null tensor");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == QS_DTYPE_BF16 && ff % 8 == 0 && out_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(in) & 15) == 0) {
    gelu_tanh_mul_bf16x8_kernel<<<dim3(tokens_n, (ff / 8 + 255) / 256), 256, 0, s>>>((__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)in, ff);
    return check_cuda(cudaGetLastError(), "hyb_gelu_tanh_mul");
  }
  dim3 grid(tokens_n, (ff + 255) / 256);
  QS_DT(dtype, (gelu_tanh_mul_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)in, ff)),
        (gelu_tanh_mul_kernel<float><<<grid, 256, 0, s>>>((float*)out, out_stride, (const float*)in, ff)));
  return check_cuda(cudaGetLastError(), "hyb_gelu_tanh_mul");
}

int qs_hyb_rope_append(void* proj, int64_t stride, const int32_t* tok_slot, const int32_t* tok_pos, const int32_t* block_table, int max_blocks,
                       void* kpool, void* vpool, const float* inv_freq, float amplitude, int tokens_n, int heads, int kv_heads, int maps,
                       int dim, int vdim, int rot_dims, int page_size, int dtype, void* stream) {
  QS_REQUIRE(proj && tok_slot && tok_pos && block_table && kpool && vpool && inv_freq, "hyb_rope_append: null tensor");
  QS_REQUIRE(rot_dims % 2 == 0 && rot_dims <= dim && heads % kv_heads == 0 && page_size > 0, "hyb_rope_append: bad head geometry");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(tokens_n, heads + kv_heads);
  QS_DT(dtype,
        (rope_append_kernel<__nv_bfloat16><<<grid, 64, 0, s>>>((__nv_bfloat16*)proj, stride, tok_slot, tok_pos, block_table, max_blocks,
                                                                (__nv_bfloat16*)kpool, (__nv_bfloat16*)vpool, inv_freq, amplitude, heads, kv_heads,
                                                                maps, dim, vdim, rot_dims, page_size)),
        (rope_append_kernel<float><<<grid, 64, 0, s>>>((float*)proj, stride, tok_slot, tok_pos, block_table, max_blocks, (float*)kpool,
                                                        (float*)vpool, inv_freq, amplitude, heads, kv_heads, maps, dim, vdim, rot_dims, page_size)));
  return check_cuda(cudaGetLastError(), "hyb_rope_append");
}

int qs_hyb_attention(void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* kpool, const void* vpool,
                     const int32_t* tok_slot, const int32_t* tok_pos, const int32_t* block_table, int max_blocks, int tokens_n, int heads,
                     int kv_heads, int maps, int dim, int vdim, float scale, float lambda, float out_scale, float eps, int head_norm,
                     int page_size, int chunk, int window, const float* sinks, const qs_attn_extra* extra, int dtype, void* stream) {
  QS_REQUIRE(out && q && kpool && vpool && tok_slot && tok_pos && block_table, "hyb_attention: null tensor");
  QS_REQUIRE(chunk >= 0 && window >= 0, "hyb_attention: negative chunk or window");
  const AttnExtra ex = attn_extra(extra);
  QS_REQUIRE(ex.keep_first >= 0 && (ex.keep_first == 0 || (window > 0 && chunk == 0)), "hyb_attention: kept first positions go with a window and no chunks");
  QS_REQUIRE(maps == 1 || maps == 2, "hyb_attention: 1 or 2 softmax maps per head");
  QS_REQUIRE(heads % kv_heads == 0 && vdim <= kAttnThreads * kAttnMaxV && page_size > 0, "hyb_attention: bad head geometry (vdim <= 512)");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  QS_DT(dtype,
        return launch_attention<__nv_bfloat16>(out, out_stride, q, q_stride, kpool, vpool, tok_slot, tok_pos, block_table, max_blocks, tokens_n,
                                               heads, kv_heads, maps, dim, vdim, scale, lambda, out_scale, eps, head_norm, page_size, chunk, window, sinks, ex, s),
        return launch_attention<float>(out, out_stride, q, q_stride, kpool, vpool, tok_slot, tok_pos, block_table, max_blocks, tokens_n, heads,
                                       kv_heads, maps, dim, vdim, scale, lambda, out_scale, eps, head_norm, page_size, chunk, window, sinks, ex, s));
}

int qs_hyb_attention_fast_supported(int dtype, int heads, int kv_heads, int maps, int dim, int vdim, int64_t q_stride) {
  return fast_attention_supported(dtype, heads, kv_heads, maps, dim, vdim, q_stride) ? 1 : 0;
}

int64_t qs_hyb_attention_scratch_floats(int tokens, int heads, int kv_heads, int maps, int vdim) {
  // per-map outputs of the tiles [tokens][heads][maps][vdim], then the single tokens' shares [tokens][heads][maps][shares][2 + vdim]
  const int64_t per = std::max(1, kv_heads * maps);
  const int64_t rows = (int64_t)tokens + (kGroupTargetBlocks + per - 1) / per;  // tokens x shares never exceeds this
  return (int64_t)tokens * heads * maps * vdim + rows * heads * maps * (2 + vdim);
}

int qs_hyb_attention_fast(void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* kpool, const void* vpool,
                          const int32_t* tok_slot, const int32_t* tok_pos, const int32_t* block_table, int max_blocks, const int32_t* tile_entry,
                          const int32_t* tile_row0, int n_tiles, const int32_t* long_tokens, int n_long, const int32_t* short_tokens, int n_short,
                          const int32_t* entry_start, const int32_t* entry_len, const int32_t* entry_slot, const int32_t* entry_pos0,
                          float* scratch, int heads, int kv_heads, int maps, int dim, int vdim, float scale, float lambda, float out_scale, float eps,
                          int head_norm, int page_size, int chunk, int window, const float* sinks, const qs_attn_extra* extra, int dtype,
                          void* stream) {
  QS_REQUIRE(chunk >= 0 && window >= 0, "hyb_attention_fast: negative chunk or window");
  const AttnExtra ex = attn_extra(extra);
  QS_REQUIRE(ex.keep_first >= 0 && (ex.keep_first == 0 || (window > 0 && chunk == 0)), "hyb_attention_fast: kept first positions go with a window and no chunks");
  QS_REQUIRE(out && q && kpool && vpool && tok_slot && tok_pos && block_table, "hyb_attention_fast: null tensor");
  QS_REQUIRE(fast_attention_supported(dtype, heads, kv_heads, maps, dim, vdim, q_stride), "hyb_attention_fast: shape not supported (use qs_hyb_attention)");
  QS_REQUIRE(n_tiles == 0 || (tile_entry && tile_row0 && long_tokens && scratch && entry_start && entry_len && entry_slot && entry_pos0),
             "hyb_attention_fast: null tile table");
  QS_REQUIRE(n_short == 0 || (short_tokens && scratch), "hyb_attention_fast: null token list");
  cudaStream_t s = (cudaStream_t)stream;
  if (n_tiles > 0) {
    int rc = 0;
#define QS_TILES(NVT, KT) rc = launch_tiles<NVT, KT>(scratch, q, q_stride, kpool, vpool, tile_entry, tile_row0, n_tiles, entry_start, entry_len, entry_slot, \
                                             entry_pos0, block_table, max_blocks, heads, kv_heads, maps, dim, scale, page_size, chunk, window, sinks, ex, s)
    switch (vdim / 16) {
      case 2: QS_TILES(2, kTileKeysPrompt); break;
      case 4: QS_TILES(4, kTileKeysPrompt); break;
      case 6: QS_TILES(6, kTileKeysPrompt); break;
      case 8: QS_TILES(8, kTileKeysPrompt); break;
      default: QS_TILES(16, 64); break;  // 128 accumulator registers: two blocks per SM either way
    }
#undef QS_TILES
    if (rc) return rc;
    const int warps = n_long * heads;
    multimap_combine_kernel<__nv_bfloat16><<<(warps + 3) / 4, 128, 0, s>>>((__nv_bfloat16*)out, out_stride, scratch, long_tokens, n_long, heads, maps, vdim,
                                                                          lambda, out_scale, eps, head_norm, (const __nv_bfloat16*)ex.gate, ex.gate_stride);
  }
  if (n_short > 0) {
    int rc = 0;
    float* part = scratch + (size_t)(n_long + n_short) * heads * maps * vdim;  // behind the per-map outputs of the tiles
#define QS_GROUP(NVT) rc = launch_group<NVT>(out, out_stride, part, q, q_stride, kpool, vpool, short_tokens, n_short, tok_slot, tok_pos, block_table, \
                                             max_blocks, heads, kv_heads, maps, dim, scale, lambda, out_scale, eps, head_norm, page_size, chunk, window, sinks, ex, s)
    switch (vdim / 16) {
      case 2: QS_GROUP(2); break;
      case 4: QS_GROUP(4); break;
      case 6: QS_GROUP(6); break;
      case 8: QS_GROUP(8); break;
      default: QS_GROUP(16); break;
    }
#undef QS_GROUP
    if (rc) return rc;
  }
  return check_cuda(cudaGetLastError(), "hyb_attention_fast");
}

int qs_hyb_gated_delta(void* out, int64_t out_stride, float* prep, float* o_raw, const void* proj, int64_t stride, const float* conv_w,
                       float* conv_state, float* state, const float* a_log, const float* dt_bias, const float* norm_w,
                       const int32_t* tok_entry, const int32_t* tok_pos, const int32_t* entry_start, const int32_t* entry_len,
                       const int32_t* entry_slot, const int32_t* entry_pos0, int tokens_n, int entries, int heads, int kv_heads, int dim,
                       int vdim, int taps, float unit_eps, float eps, int dtype, void* stream) {
  QS_REQUIRE(out && prep && o_raw && proj && conv_w && state && a_log && dt_bias && norm_w, "hyb_gated_delta: null tensor");
  QS_REQUIRE(tok_entry && tok_pos && entry_start && entry_len && entry_slot && entry_pos0, "hyb_gated_delta: null batch table");
  QS_REQUIRE(taps >= 1 && taps <= 17 && (taps == 1 || conv_state != nullptr), "hyb_gated_delta: 1..17 convolution taps");
  QS_REQUIRE(heads % kv_heads == 0 && dim <= 256 && vdim <= 1024, "hyb_gated_delta: dim <= 256, vdim <= 1024");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  QS_DT(dtype,
        return launch_delta<__nv_bfloat16>(out, out_stride, prep, o_raw, proj, stride, conv_w, conv_state, state, a_log, dt_bias, norm_w,
                                           tok_entry, tok_pos, entry_start, entry_len, entry_slot, entry_pos0, tokens_n, entries, heads,
                                           kv_heads, dim, vdim, taps, unit_eps, eps, s),
        return launch_delta<float>(out, out_stride, prep, o_raw, proj, stride, conv_w, conv_state, state, a_log, dt_bias, norm_w, tok_entry,
                                   tok_pos, entry_start, entry_len, entry_slot, entry_pos0, tokens_n, entries, heads, kv_heads, dim, vdim,
                                   taps, unit_eps, eps, s));
}

}  // extern "C"
