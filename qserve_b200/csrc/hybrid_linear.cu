// qserve_b200 -- linear recurrences of the hybrid decoders: per head a [D, Dv] fp32 state that every token decays, writes to and reads.
//
//   gate recurrence (HGRN2):  S <- diag(f) S + (1 - f) v^T,  o = S^T q      f per (head, row): the forget gate also sets the write strength
//   retention:                S <- decay_h S + k v^T,        o = S^T q      one fixed decay per head, rotary q / k
//   gated linear attention:   S <- diag(a) S + k v^T,        o = S^T q      a per (head, row) from a low-rank projection of the input
//
// Both run in three steps on the flat token batch (hybrid.cu describes the batch tables):
//   1. prepare: projection rows -> fp32 rows [H*D q | H*D g | H*Dv v]  (g = f, or the rotated and scaled k; gated linear attention has
//      three row vectors: [H*D q | H*D k | H*D a | H*Dv v]); everything that enters the recurrence is fp32 from here on
//   2. scan: one block per (entry, head, block of state columns) walks the entry's tokens in order with its columns of S in registers; a run
//      that starts at position 0 starts from zero, the others from the state slot; the slot takes the state after the run
//   3. read-out: per (token, head) unit RMS [times a per-dimension gain] [times silu(output gate)] -> storage type
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
// step 1, gate recurrence.  projection row: [H*D q | H*D f | H*Dv v];  q <- silu(q),  f <- lower + (1 - lower) sigmoid(f + bias)
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename ST>
__global__ void gate_prepare_kernel(float* __restrict__ prep, const ST* __restrict__ proj, long long stride, const float* __restrict__ f_bias,
                                    const float* __restrict__ lower, int HD, int HDv) {
  const int t = blockIdx.x;
  const ST* row = proj + (size_t)t * stride;
  float* o = prep + (size_t)t * (2 * HD + HDv);
  for (int c = threadIdx.x; c < 2 * HD + HDv; c += blockDim.x) {
    const float x = ldf(row + c);
    float y = x;
    if (c < HD) {
      y = silu_f(x);
    } else if (c < 2 * HD) {
      const float lo = lower[c - HD];
      y = lo + (1.f - lo) * (1.f / (1.f + expf(-(x + f_bias[c - HD]))));
    }
    o[c] = y;
  }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// step 1, retention.  projection row: [H*D q | H*D k | H*Dv v | ...];  q and k are rotated on their first rot_dims entries (entry i is paired
// with entry i + rot_dims/2, angle = position * inv_freq[i]), k is then scaled by k_scale
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename ST>
__global__ void retention_prepare_kernel(float* __restrict__ prep, const ST* __restrict__ proj, long long stride, const int* __restrict__ tok_pos,
                                         const float* __restrict__ inv_freq, int rot_dims, float k_scale, int H, int D, int Dv) {
  extern __shared__ float cs[];  // cos [rot_dims / 2] | sin [rot_dims / 2] of the token's position: one evaluation serves q and k of every head
  const int t = blockIdx.x;
  const int HD = H * D, half = rot_dims >> 1;
  const float pos = (float)tok_pos[t];
  for (int p = threadIdx.x; p < half; p += blockDim.x) sincosf(pos * inv_freq[p], &cs[half + p], &cs[p]);
  __syncthreads();
  const ST* row = proj + (size_t)t * stride;
  float* o = prep + (size_t)t * (2 * HD + H * Dv);
  for (int c = threadIdx.x; c < 2 * HD + H * Dv; c += blockDim.x) {
    float y = ldf(row + c);
    if (c < 2 * HD) {
      const int d = c % D;
      if (d < rot_dims) {
        const bool first = d < half;
        const float other = ldf(row + (first ? c + half : c - half));
        const int p = first ? d : d - half;
        y = first ? y * cs[p] - other * cs[half + p] : y * cs[p] + other * cs[half + p];
      }
      if (c >= HD) y *= k_scale;
    }
    o[c] = y;
  }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// step 1, gated linear attention.  projection row: [H*D q | H*D k | H*Dv v | ...]; z fp32 [tokens, H*D]: the decay logits before their bias.
//   q <- q * q_scale;   a = sigmoid(z + bias)^(1/tau) = exp(log_sigmoid(z + bias) / tau), log_sigmoid(u) = min(u, 0) - log1p(exp(-|u|))
// prepared row: [H*D q | H*D k | H*D a | H*Dv v]
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename ST>
__global__ void gated_linear_prepare_kernel(float* __restrict__ prep, const ST* __restrict__ proj, long long stride, const float* __restrict__ z,
                                            const float* __restrict__ z_bias, float inv_tau, float q_scale, int HD, int HDv) {
  const int t = blockIdx.x;
  const ST* row = proj + (size_t)t * stride;
  float* o = prep + (size_t)t * (3 * HD + HDv);
  for (int c = threadIdx.x; c < 2 * HD; c += blockDim.x) o[c] = c < HD ? ldf(row + c) * q_scale : ldf(row + c);
  for (int c = threadIdx.x; c < HD; c += blockDim.x) {
    const float u = z[(size_t)t * HD + c] + (z_bias != nullptr ? z_bias[c] : 0.f);
    o[2 * HD + c] = expf((fminf(u, 0.f) - log1pf(expf(-fabsf(u)))) * inv_tau);
  }
  for (int c = threadIdx.x; c < HDv; c += blockDim.x) o[3 * HD + c] = ldf(row + 2 * HD + c);
}

// ---------------------------------------------------------------------------------------------------------------------------------
// step 2.  Columns of a head's [D, Dv] state are independent, so a block owns 128 / PARTS columns of one (entry, head): thread (column, part)
// keeps rows [part Q, (part + 1) Q) of its column in registers (Q = DP / PARTS, D <= DP); the parts of a column sit in adjacent lanes and meet
// through shuffles.  Tokens are staged CH at a time (q | g | v of the block's columns) with cp.async into a double buffer, so that no global
// load sits on the token-to-token dependency chain.
//   MODE kScanHeadDecay:    S_i <- decay S_i + g_i v
//   MODE kScanChannelGate:  S_i <- g_i S_i + (1 - g_i) v   (written as v + g_i (S_i - v))
//   MODE kScanChannelDecay: S_i <- a_i S_i + g_i v         (a third row vector a follows g in the prepared row)
//   o = sum_i S_i q_i
// ---------------------------------------------------------------------------------------------------------------------------------
template <int PARTS>
__device__ __forceinline__ float part_sum(float v) {
#pragma unroll
  for (int o = 1; o < PARTS; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int kScanHeadDecay = 0, kScanChannelGate = 1, kScanChannelDecay = 2;

template <int DP, int PARTS, int CH, int CPT, int MODE, bool VEC>  // VEC: 16-byte staging (D, Dv, the prepared row and its base allow it)
__global__ void __launch_bounds__(128) linear_scan_kernel(float* __restrict__ o_raw, const float* __restrict__ prep, float* __restrict__ state,
                                                          const float* __restrict__ head_decay, const int* __restrict__ entry_start,
                                                          const int* __restrict__ entry_len, const int* __restrict__ entry_slot,
                                                          const int* __restrict__ entry_pos0, int H, int D, int Dv) {
  extern __shared__ __align__(16) float sm[];  // [2][CH][ROW]
  constexpr int Q = DP / PARTS, SEG = Q + 4, COLS = 128 / PARTS * CPT;  // a part's q / g segment is padded by 16 bytes: parts hit different banks
  constexpr int NVEC = MODE == kScanChannelDecay ? 3 : 2;  // row vectors of a token: q, g [, a]
  constexpr int QK = PARTS * SEG, ROW = NVEC * QK + COLS;
  const int e = blockIdx.x, h = blockIdx.y, cg = blockIdx.z;
  const int tid = threadIdx.x, part = tid % PARTS, cl = tid / PARTS, col0 = cg * COLS + cl * CPT;  // CPT adjacent columns per thread
  const int HD = H * D, P = NVEC * HD + H * Dv;
  const int n = entry_len[e], s0 = entry_start[e];
  const bool fresh = entry_pos0[e] == 0;
  const float decay = MODE == kScanHeadDecay ? head_decay[h] : 0.f;
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
      constexpr int QV = Q / 4, NQK = NVEC * PARTS * QV, NV = COLS / 4, ITEMS = NQK + NV;
      for (int idx = tid; idx < CH * ITEMS; idx += 128) {
        const int tk = idx / ITEMS, j = idx - tk * ITEMS, t = chunk * CH + tk;
        float* base = sm + (size_t)(buf * CH + tk) * ROW;
        const float* row = prep + (size_t)(s0 + min(t, n - 1)) * P;
        float* dst;
        const float* src = nullptr;
        if (j < NQK) {
          const int which = j / (PARTS * QV), rem = j - which * (PARTS * QV), pp = rem / QV, w4 = rem - pp * QV, i = pp * Q + w4 * 4;
          dst = base + which * QK + pp * SEG + w4 * 4;
          if (i < D) src = row + (size_t)which * HD + (size_t)h * D + i;
        } else {
          const int c4 = (j - NQK) * 4, c = cg * COLS + c4;
          dst = base + NVEC * QK + c4;
          if (c < Dv) src = row + NVEC * HD + (size_t)h * Dv + c;
        }
        if (t < n && src != nullptr) cp_async16(dst, src);
        else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
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
        if (j < NVEC * QK) {
          const int which = j / QK, jj = j - which * QK, pp = jj / SEG, w = jj - pp * SEG, i = pp * Q + w;  // q (which = 0), g or a row i
          if (w < Q && i < D) src = row + (size_t)which * HD + (size_t)h * D + i;
        } else {
          const int c = cg * COLS + j - NVEC * QK;
          if (c < Dv) src = row + NVEC * HD + (size_t)h * Dv + c;
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
      const float4* g4 = reinterpret_cast<const float4*>(r + QK + part * SEG);
      const float4* a4 = reinterpret_cast<const float4*>(r + (NVEC - 1) * QK + part * SEG);  // read in kScanChannelDecay only
      float v[CPT], op[CPT][4];
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        v[c] = r[NVEC * QK + cl * CPT + c];
        op[c][0] = op[c][1] = op[c][2] = op[c][3] = 0.f;
      }
      // a q / g word read from shared memory serves the thread's CPT columns
#pragma unroll
      for (int j = 0; j < Q / 4; ++j) {
        const float4 gg = g4[j], qq = q4[j];
        float4 aa = make_float4(decay, decay, decay, decay);
        if (MODE == kScanChannelDecay) aa = a4[j];
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          float* Sc = S[c];
          if (MODE == kScanChannelGate) {
            Sc[4 * j] = v[c] + gg.x * (Sc[4 * j] - v[c]);
            Sc[4 * j + 1] = v[c] + gg.y * (Sc[4 * j + 1] - v[c]);
            Sc[4 * j + 2] = v[c] + gg.z * (Sc[4 * j + 2] - v[c]);
            Sc[4 * j + 3] = v[c] + gg.w * (Sc[4 * j + 3] - v[c]);
          } else {
            Sc[4 * j] = Sc[4 * j] * aa.x + gg.x * v[c];
            Sc[4 * j + 1] = Sc[4 * j + 1] * aa.y + gg.y * v[c];
            Sc[4 * j + 2] = Sc[4 * j + 2] * aa.z + gg.z * v[c];
            Sc[4 * j + 3] = Sc[4 * j + 3] * aa.w + gg.w * v[c];
          }
          op[c][0] += Sc[4 * j] * qq.x; op[c][1] += Sc[4 * j + 1] * qq.y; op[c][2] += Sc[4 * j + 2] * qq.z; op[c][3] += Sc[4 * j + 3] * qq.w;
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

// step 3: per (token, head): o * rsqrt(mean(o^2) + eps) [* norm_w] [* silu(gate)]; one warp each.  gate: storage-type rows of `stride`
// elements whose entry h * Dv + i gates output i of head h
template <typename ST>
__global__ void linear_out_kernel(ST* __restrict__ out, long long out_stride, const float* __restrict__ o_raw, const float* __restrict__ norm_w,
                                  const ST* __restrict__ gate, long long stride, int T, int H, int Dv, float eps) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= T * H) return;
  const int t = w / H, h = w - t * H;
  const float* o = o_raw + (size_t)t * H * Dv + (size_t)h * Dv;
  float ss = 0.f;
  for (int i = lane; i < Dv; i += 32) ss += o[i] * o[i];
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)Dv + eps);
  ST* dst = out + (size_t)t * out_stride + (size_t)h * Dv;
  for (int i = lane; i < Dv; i += 32) {
    float y = o[i] * r;
    if (norm_w != nullptr) y *= norm_w[i];
    if (gate != nullptr) y *= silu_f(ldf(gate + (size_t)t * stride + (size_t)h * Dv + i));
    stf(dst + i, y);
  }
}

template <int MODE>
int launch_scan(float* o_raw, const float* prep, float* state, const float* head_decay, const int* entry_start, const int* entry_len,
                const int* entry_slot, const int* entry_pos0, int T, int E, int H, int D, int Dv, cudaStream_t s) {
  constexpr int NVEC = MODE == kScanChannelDecay ? 3 : 2;
  const int P = NVEC * H * D + H * Dv;
  const bool vec = D % 4 == 0 && Dv % 4 == 0 && P % 4 == 0 && (reinterpret_cast<uintptr_t>(prep) & 15) == 0;
#define QS_SCAN(DP, PARTS, CH, CPT)                                                                                                           \
  do {                                                                                                                                        \
    constexpr int cols = 128 / PARTS * CPT;                                                                                                   \
    const size_t smb = (size_t)2 * CH * (NVEC * PARTS * (DP / PARTS + 4) + cols) * sizeof(float);                                                \
    dim3 grid(E, H, (Dv + cols - 1) / cols);                                                                                                  \
    auto kern = vec ? linear_scan_kernel<DP, PARTS, CH, CPT, MODE, true> : linear_scan_kernel<DP, PARTS, CH, CPT, MODE, false>;                 \
    if (smb > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smb);                                   \
    kern<<<grid, 128, smb, s>>>(o_raw, prep, state, head_decay, entry_start, entry_len, entry_slot, entry_pos0, H, D, Dv);                    \
  } while (0)
  // rows of a column per thread: all of them up to 32, 32 or 16 above (the parts of a column meet through shuffles).  Long runs of tokens
  // (prompt portions) take two adjacent columns per thread where the head has the columns for it: a q / g word read from shared memory then
  // feeds two columns; steps of mostly single tokens are bound by reading and writing the state and keep one column per thread
  const bool long_runs = T >= 32 * E;
  if (D <= 16) QS_SCAN(16, 1, 16, 1);
  else if (D <= 32) QS_SCAN(32, 1, 16, 1);
  else if (D <= 64) { if (Dv >= 128 && long_runs) QS_SCAN(64, 2, 16, 2); else QS_SCAN(64, 2, 16, 1); }
  // (three row vectors per token: chunks of 8 tokens keep a block's staging near 32 KB, so that as many blocks share an SM as with two)
  else if (D <= 128) {
    if (Dv >= 64 && long_runs) { if (NVEC == 3) QS_SCAN(128, 8, 8, 2); else QS_SCAN(128, 8, 16, 2); }
    else QS_SCAN(128, 4, 16, 1);
  }
  else if (D <= 256) QS_SCAN(256, 8, 8, 1);
  else QS_SCAN(512, 16, 4, 1);
#undef QS_SCAN
  return check_cuda(cudaGetLastError(), "hyb linear scan");
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

int qs_hyb_gate_recurrence(void* out, int64_t out_stride, float* prep, float* o_raw, const void* proj, int64_t stride, const float* f_bias,
                           const float* lower, const float* norm_w, float* state, const int32_t* entry_start, const int32_t* entry_len,
                           const int32_t* entry_slot, const int32_t* entry_pos0, int tokens_n, int entries, int heads, int dim, int vdim,
                           float eps, int dtype, void* stream) {
  QS_REQUIRE(out && prep && o_raw && proj && f_bias && lower && state, "hyb_gate_recurrence: null tensor");
  QS_REQUIRE(entry_start && entry_len && entry_slot && entry_pos0, "hyb_gate_recurrence: null batch table");
  QS_REQUIRE(heads > 0 && dim > 0 && dim <= 512 && vdim > 0, "hyb_gate_recurrence: 0 < dim <= 512");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int HD = heads * dim, HDv = heads * vdim;
  QS_DT(dtype, (gate_prepare_kernel<__nv_bfloat16><<<tokens_n, 256, 0, s>>>(prep, (const __nv_bfloat16*)proj, stride, f_bias, lower, HD, HDv)),
        (gate_prepare_kernel<float><<<tokens_n, 256, 0, s>>>(prep, (const float*)proj, stride, f_bias, lower, HD, HDv)));
  if (int rc = launch_scan<kScanChannelGate>(o_raw, prep, state, nullptr, entry_start, entry_len, entry_slot, entry_pos0, tokens_n, entries, heads, dim, vdim, s)) return rc;
  const int warps = tokens_n * heads;
  QS_DT(dtype,
        (linear_out_kernel<__nv_bfloat16><<<(warps + 3) / 4, 128, 0, s>>>((__nv_bfloat16*)out, out_stride, o_raw, norm_w, nullptr, 0, tokens_n, heads,
                                                                           vdim, eps)),
        (linear_out_kernel<float><<<(warps + 3) / 4, 128, 0, s>>>((float*)out, out_stride, o_raw, norm_w, nullptr, 0, tokens_n, heads, vdim, eps)));
  return check_cuda(cudaGetLastError(), "hyb_gate_recurrence");
}

int qs_hyb_retention(void* out, int64_t out_stride, float* prep, float* o_raw, const void* proj, int64_t stride, const float* head_decay,
                     const float* inv_freq, int rot_dims, float k_scale, int gated, float* state, const int32_t* tok_pos,
                     const int32_t* entry_start, const int32_t* entry_len, const int32_t* entry_slot, const int32_t* entry_pos0, int tokens_n,
                     int entries, int heads, int dim, int vdim, float eps, int dtype, void* stream) {
  QS_REQUIRE(out && prep && o_raw && proj && head_decay && state && tok_pos, "hyb_retention: null tensor");
  QS_REQUIRE(entry_start && entry_len && entry_slot && entry_pos0, "hyb_retention: null batch table");
  QS_REQUIRE(heads > 0 && dim > 0 && dim <= 512 && vdim > 0, "hyb_retention: 0 < dim <= 512");
  QS_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dim && (rot_dims == 0 || inv_freq != nullptr), "hyb_retention: bad rotary size");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  QS_DT(dtype,
        (retention_prepare_kernel<__nv_bfloat16><<<tokens_n, 256, rot_dims * sizeof(float), s>>>(prep, (const __nv_bfloat16*)proj, stride, tok_pos, inv_freq, rot_dims, k_scale,
                                                                           heads, dim, vdim)),
        (retention_prepare_kernel<float><<<tokens_n, 256, rot_dims * sizeof(float), s>>>(prep, (const float*)proj, stride, tok_pos, inv_freq, rot_dims, k_scale, heads, dim,
                                                                  vdim)));
  if (int rc = launch_scan<kScanHeadDecay>(o_raw, prep, state, head_decay, entry_start, entry_len, entry_slot, entry_pos0, tokens_n, entries, heads, dim, vdim, s)) return rc;
  const int warps = tokens_n * heads;
  const size_t gate_off = (size_t)2 * heads * dim + (size_t)heads * vdim;  // the output gate follows q | k | v in the projection row
  QS_DT(dtype,
        (linear_out_kernel<__nv_bfloat16><<<(warps + 3) / 4, 128, 0, s>>>((__nv_bfloat16*)out, out_stride, o_raw, nullptr,
                                                                           gated ? (const __nv_bfloat16*)proj + gate_off : nullptr, stride, tokens_n,
                                                                           heads, vdim, eps)),
        (linear_out_kernel<float><<<(warps + 3) / 4, 128, 0, s>>>((float*)out, out_stride, o_raw, nullptr, gated ? (const float*)proj + gate_off : nullptr,
                                                                  stride, tokens_n, heads, vdim, eps)));
  return check_cuda(cudaGetLastError(), "hyb_retention");
}

int qs_hyb_gated_linear(void* out, int64_t out_stride, float* prep, float* o_raw, const void* proj, int64_t stride, const float* z, const float* z_bias,
                        float tau, const float* norm_w, float* state, const int32_t* entry_start, const int32_t* entry_len, const int32_t* entry_slot,
                        const int32_t* entry_pos0, int tokens_n, int entries, int heads, int dim, int vdim, float eps, int dtype, void* stream) {
  QS_REQUIRE(out && prep && o_raw && proj && z && state, "hyb_gated_linear: null tensor");
  QS_REQUIRE(entry_start && entry_len && entry_slot && entry_pos0, "hyb_gated_linear: null batch table");
  QS_REQUIRE(heads > 0 && dim > 0 && dim <= 512 && vdim > 0 && tau > 0.f, "hyb_gated_linear: 0 < dim <= 512, tau > 0");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int HD = heads * dim, HDv = heads * vdim;
  const float inv_tau = 1.f / tau, q_scale = 1.f / sqrtf((float)dim);
  QS_DT(dtype,
        (gated_linear_prepare_kernel<__nv_bfloat16><<<tokens_n, 256, 0, s>>>(prep, (const __nv_bfloat16*)proj, stride, z, z_bias, inv_tau, q_scale, HD, HDv)),
        (gated_linear_prepare_kernel<float><<<tokens_n, 256, 0, s>>>(prep, (const float*)proj, stride, z, z_bias, inv_tau, q_scale, HD, HDv)));
  if (int rc = launch_scan<kScanChannelDecay>(o_raw, prep, state, nullptr, entry_start, entry_len, entry_slot, entry_pos0, tokens_n, entries, heads, dim, vdim, s)) return rc;
  const int warps = tokens_n * heads;
  const size_t gate_off = (size_t)2 * HD + (size_t)HDv;  // the output gate follows q | k | v in the projection row
  QS_DT(dtype,
        (linear_out_kernel<__nv_bfloat16><<<(warps + 3) / 4, 128, 0, s>>>((__nv_bfloat16*)out, out_stride, o_raw, norm_w, (const __nv_bfloat16*)proj + gate_off,
                                                                           stride, tokens_n, heads, vdim, eps)),
        (linear_out_kernel<float><<<(warps + 3) / 4, 128, 0, s>>>((float*)out, out_stride, o_raw, norm_w, (const float*)proj + gate_off, stride, tokens_n, heads,
                                                                  vdim, eps)));
  return check_cuda(cudaGetLastError(), "hyb_gated_linear");
}

}  // extern "C"
