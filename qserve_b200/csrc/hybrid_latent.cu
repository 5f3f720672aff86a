// qserve_b200 -- latent attention of the hybrid decoders: keys and values of all heads are linear images of one small latent row per
// position, so the paged cache holds only that row and one rotated key part shared by the heads:
//
//   cell [page][page_size][K + R]:  c = rms_norm(W_dkv h)[0:K] * gain      |  k_rot = rotate(W_dkv h)[K:K+R]
//
// The scores of head h are (q_h^nope . W_uk,h c + q_h^rot . k_rot) * scale.  W_uk,h is moved to the query side (q_h^lat = W_uk,h^T q_h^nope,
// a batched matrix product), so a head's query becomes a row of K + R numbers that is scored against the cached cell as it lies in memory;
// the weighted sum of the cells' first K numbers is taken up to the head's values by W_uv,h afterwards (another batched product).  In this
// form every head reads the same K + R numbers per position: the cache traffic of a step does not grow with the number of heads.
//
// Kernels: latent_prepare (norms of both latents, rotation of the shared key part, append to the pages), latent_query (rotation of the
// query's rotated part, assembly of the K + R query rows), latent_attention (any shape, fp32 or bfloat16 storage, CUDA cores),
// latent_tile_attention (bfloat16 storage on the tensor cores: the rows of a tile are (token, head) pairs of one sequence),
// latent_gate_out (head-major value rows times a sigmoid gate per head into the rows of the output projection).
// The flat token batch (per-token slot and position tables, block table) is described in hybrid.cu.
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
// One block per token.  Row of the first projection: [col_q, col_q + Q): query latent, [col_kv, col_kv + K + R): key/value latent and the
// shared rotated key part.
//   cq[t] = row_q * rsqrt(mean(row_q^2) + eps) * gain_q                         (storage type, feeds the query up-projection)
//   cell  = [row_c * rsqrt(mean(row_c^2) + eps) * gain_kv | rotate(row_r)]      (storage type, in the token's page)
// Rotation ("half" layout): entry i < dims/2 is paired with entry i + dims/2, angle = position * inv_freq[i]; entries from `dims` on pass.
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename ST>
__global__ void __launch_bounds__(128) latent_prepare_kernel(ST* __restrict__ cq, const ST* __restrict__ proj, long long stride, int col_q, int col_kv,
                                                             const float* __restrict__ gain_q, const float* __restrict__ gain_kv,
                                                             const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ tok_slot,
                                                             const int* __restrict__ tok_pos, const int* __restrict__ block_table, int max_blocks,
                                                             ST* __restrict__ pool, int Q, int K, int R, int page, float eps) {
  __shared__ float red[33];
  const int t = blockIdx.x, tid = threadIdx.x;
  const ST* row = proj + (size_t)t * stride;
  const int pos = tok_pos[t];
  float sq = 0.f, sk = 0.f;
  for (int i = tid; i < Q; i += blockDim.x) {
    const float v = ldf(row + col_q + i);
    sq += v * v;
  }
  for (int i = tid; i < K; i += blockDim.x) {
    const float v = ldf(row + col_kv + i);
    sk += v * v;
  }
  sq = block_sum(sq, red);
  sk = block_sum(sk, red);
  const float rq = 1.f / sqrtf(sq / (float)Q + eps), rk = 1.f / sqrtf(sk / (float)K + eps);
  for (int i = tid; i < Q; i += blockDim.x) stf(cq + (size_t)t * Q + i, ldf(row + col_q + i) * rq * gain_q[i]);
  const int pg = block_table[(size_t)tok_slot[t] * max_blocks + pos / page];
  ST* cell = pool + ((size_t)pg * page + pos % page) * (size_t)(K + R);
  for (int i = tid; i < K; i += blockDim.x) stf(cell + i, ldf(row + col_kv + i) * rk * gain_kv[i]);
  const ST* kr = row + col_kv + K;
  const int half = rot_dims >> 1;
  for (int i = tid; i < R; i += blockDim.x) {
    float v = ldf(kr + i);
    if (i < rot_dims) {
      const int p = i < half ? i : i - half;
      float s, c;
      sincosf((float)pos * inv_freq[p], &s, &c);
      const float a = ldf(kr + p), b = ldf(kr + p + half);
      v = i < half ? a * c - b * s : b * c + a * s;
    }
    stf(cell + K + i, v);
  }
}

// query rows of K + R numbers: qa[t][h] = [qlat[h][t][0:K] | rotate(q[t][h][D : D + R])].  One block per (token, head).
template <typename ST>
__global__ void __launch_bounds__(64) latent_query_kernel(ST* __restrict__ qa, const ST* __restrict__ qlat, const ST* __restrict__ q, long long q_stride,
                                                          const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ tok_pos, int T, int H,
                                                          int D, int K, int R) {
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  ST* dst = qa + ((size_t)t * H + h) * (size_t)(K + R);
  const ST* src = qlat + ((size_t)h * T + t) * (size_t)K;
  for (int i = tid; i < K; i += blockDim.x) dst[i] = src[i];
  const ST* qr = q + (size_t)t * q_stride + (size_t)h * (D + R) + D;
  const int pos = tok_pos[t], half = rot_dims >> 1;
  for (int i = tid; i < R; i += blockDim.x) {
    float v = ldf(qr + i);
    if (i < rot_dims) {
      const int p = i < half ? i : i - half;
      float s, c;
      sincosf((float)pos * inv_freq[p], &s, &c);
      const float a = ldf(qr + p), b = ldf(qr + p + half);
      v = i < half ? a * c - b * s : b * c + a * s;
    }
    stf(dst + K + i, v);
  }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// Latent attention, any shape (CUDA cores, fp32 arithmetic).  One block = one token x (4 warps x HPW heads); all heads of the block score
// the same cells, so a tile of KT cells is staged in shared memory once and meets 4 HPW heads.  Per tile: lane j of a warp scores cell j for
// the warp's heads, an online softmax per head (fp32 weights), then lane c accumulates output columns c, c + 32, ... of the latent.
// Tiles start at the first visible position of the token, so a position's sums are formed in the same order however the prompt was cut and
// whatever else the batch holds.
//   out[h][t][0:K] = sum_j softmax_j(scale * qa[t][h] . cell_j) cell_j[0:K]            (head-major: the batch of the value up-projection)
// ---------------------------------------------------------------------------------------------------------------------------------
constexpr int kLatKT = 32;       // cells per tile = lanes of a warp
constexpr int kLatMaxVC = 16;    // output columns per lane: K <= 512

template <typename ST> __host__ __device__ constexpr int lat_row_stride(int dk) {
  // shared-memory row stride (elements) whose 32-bit word stride is odd: the lanes of a warp read the same column of 32 different rows
  return sizeof(ST) == 4 ? (dk | 1) : ((((dk + 1) / 2) | 1) * 2);
}

template <typename ST, int HPW>
__global__ void __launch_bounds__(128) latent_attention_kernel(ST* __restrict__ out, const ST* __restrict__ qa, const ST* __restrict__ pool,
                                                               const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
                                                               const int* __restrict__ block_table, int max_blocks, int T, int H, int K, int R,
                                                               float scale, int page, int chunk, int window) {
  extern __shared__ __align__(16) unsigned char dyn_raw[];
  const int DK = K + R, SD = lat_row_stride<ST>(DK);
  float* qs = reinterpret_cast<float*>(dyn_raw);                 // [4 HPW][DK]
  float* ps = qs + 4 * HPW * DK;                                 // [4 HPW][KT]
  ST* ks = reinterpret_cast<ST*>(ps + 4 * HPW * kLatKT);         // [KT][SD]
  __shared__ long long cells[kLatKT];
  const int t = blockIdx.x, h0 = blockIdx.y * 4 * HPW, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pos = tok_pos[t];
  const int* bt = block_table + (size_t)tok_slot[t] * max_blocks;
  for (int i = tid; i < 4 * HPW * DK; i += 128) {
    const int hh = h0 + i / DK;
    qs[i] = hh < H ? ldf(qa + ((size_t)t * H + hh) * DK + (i % DK)) : 0.f;
  }
  float m_run[HPW], l_run[HPW], acc[HPW][kLatMaxVC];
#pragma unroll
  for (int u = 0; u < HPW; ++u) {
    m_run[u] = -INFINITY;
    l_run[u] = 0.f;
#pragma unroll
    for (int i = 0; i < kLatMaxVC; ++i) acc[u][i] = 0.f;
  }
  const int n_keys = pos + 1;
  for (int base = first_key(pos, chunk, window); base < n_keys; base += kLatKT) {
    const int nk = min(kLatKT, n_keys - base);
    __syncthreads();  // the previous tile is consumed (and qs written, the first time)
    if (tid < nk) cells[tid] = (long long)bt[(base + tid) / page] * page + (base + tid) % page;
    __syncthreads();
    for (int i = tid; i < nk * DK; i += 128) {
      const int j = i / DK, d = i - j * DK;
      ks[j * SD + d] = pool[(size_t)cells[j] * DK + d];
    }
    __syncthreads();
    // scores: lane = cell
    float s[HPW];
#pragma unroll
    for (int u = 0; u < HPW; ++u) s[u] = 0.f;
    if (lane < nk) {
      const ST* kr = ks + lane * SD;
      for (int d = 0; d < DK; ++d) {
        const float kv = ldf(kr + d);
#pragma unroll
        for (int u = 0; u < HPW; ++u) s[u] += qs[(warp * HPW + u) * DK + d] * kv;
      }
    }
    float corr[HPW];
#pragma unroll
    for (int u = 0; u < HPW; ++u) {
      const float v = lane < nk ? s[u] * scale : -INFINITY;
      const float m_new = fmaxf(m_run[u], warp_max(v));
      const float p = lane < nk ? expf(v - m_new) : 0.f;
      corr[u] = expf(m_run[u] - m_new);  // 0 on the first tile
      l_run[u] = l_run[u] * corr[u] + warp_sum(p);
      m_run[u] = m_new;
      ps[(warp * HPW + u) * kLatKT + lane] = p;
    }
    __syncwarp();
    // weighted cells: lane = output column
#pragma unroll
    for (int i = 0; i < kLatMaxVC; ++i) {
      const int c = lane + 32 * i;
      if (c < K) {
        float a[HPW];
#pragma unroll
        for (int u = 0; u < HPW; ++u) a[u] = acc[u][i] * corr[u];
        for (int j = 0; j < nk; ++j) {
          const float v = ldf(ks + j * SD + c);
#pragma unroll
          for (int u = 0; u < HPW; ++u) a[u] += ps[(warp * HPW + u) * kLatKT + j] * v;
        }
#pragma unroll
        for (int u = 0; u < HPW; ++u) acc[u][i] = a[u];
      }
    }
  }
#pragma unroll
  for (int u = 0; u < HPW; ++u) {
    const int h = h0 + warp * HPW + u;
    if (h >= H) continue;
    const float inv = 1.f / l_run[u];
    ST* o = out + ((size_t)h * T + t) * (size_t)K;
#pragma unroll
    for (int i = 0; i < kLatMaxVC; ++i) {
      const int c = lane + 32 * i;
      if (c < K) stf(o + c, acc[u][i] * inv);
    }
  }
}

template <typename ST, int HPW>
int launch_latent_attention(void* out, const void* qa, const void* pool, const int* tok_slot, const int* tok_pos, const int* block_table,
                            int max_blocks, int T, int H, int K, int R, float scale, int page, int chunk, int window, cudaStream_t s) {
  const int DK = K + R;
  const size_t smem = (size_t)4 * HPW * (DK + kLatKT) * sizeof(float) + (size_t)kLatKT * lat_row_stride<ST>(DK) * sizeof(ST);
  QS_REQUIRE(smem <= 200 * 1024, "hyb_latent_attention: latent row too wide for shared memory");
  static bool attr_set[kMaxDevices] = {};
  if (smem > 48 * 1024 && !attr_set[device_ordinal()]) {
    if (int rc = check_cuda(cudaFuncSetAttribute(latent_attention_kernel<ST, HPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024),
                            "latent attention smem"))
      return rc;
    attr_set[device_ordinal()] = true;
  }
  latent_attention_kernel<ST, HPW><<<dim3(T, (H + 4 * HPW - 1) / (4 * HPW)), 128, smem, s>>>((ST*)out, (const ST*)qa, (const ST*)pool, tok_slot, tok_pos,
                                                                                          block_table, max_blocks, T, H, K, R, scale, page, chunk, window);
  return check_cuda(cudaGetLastError(), "hyb_latent_attention");
}

// out[t][h * Dv + j] = ov[h][t][j] * sigmoid(gate[t][col_g + h])   (gate == null: no gate).  One block per token.
template <typename ST>
__global__ void latent_gate_out_kernel(ST* __restrict__ out, long long out_stride, const ST* __restrict__ ov, const ST* __restrict__ gate,
                                       long long gate_stride, int col_g, int T, int H, int Dv) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < H * Dv; i += blockDim.x) {
    const int h = i / Dv, j = i - h * Dv;
    float v = ldf(ov + ((size_t)h * T + t) * Dv + j);
    if (gate != nullptr) v *= 1.f / (1.f + expf(-ldf(gate + (size_t)t * gate_stride + col_g + h)));
    stf(out + (size_t)t * out_stride + i, v);
  }
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

int qs_hyb_latent_prepare(void* cq, const void* proj, int64_t stride, int col_q, int col_kv, const float* gain_q, const float* gain_kv,
                          const float* inv_freq, int rot_dims, const int32_t* tok_slot, const int32_t* tok_pos, const int32_t* block_table,
                          int max_blocks, void* pool, int tokens_n, int q_rank, int kv_rank, int rot_dim, int page_size, float eps, int dtype,
                          void* stream) {
  QS_REQUIRE(cq && proj && gain_q && gain_kv && tok_slot && tok_pos && block_table && pool, "hyb_latent_prepare: null tensor");
  QS_REQUIRE(q_rank > 0 && kv_rank > 0 && rot_dim >= 0 && page_size > 0, "hyb_latent_prepare: bad sizes");
  QS_REQUIRE(rot_dims % 2 == 0 && rot_dims >= 0 && rot_dims <= rot_dim && (rot_dims == 0 || inv_freq), "hyb_latent_prepare: bad rotation");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  QS_DT(dtype,
        (latent_prepare_kernel<__nv_bfloat16><<<tokens_n, 128, 0, s>>>((__nv_bfloat16*)cq, (const __nv_bfloat16*)proj, stride, col_q, col_kv, gain_q,
                                                                        gain_kv, inv_freq, rot_dims, tok_slot, tok_pos, block_table, max_blocks,
                                                                        (__nv_bfloat16*)pool, q_rank, kv_rank, rot_dim, page_size, eps)),
        (latent_prepare_kernel<float><<<tokens_n, 128, 0, s>>>((float*)cq, (const float*)proj, stride, col_q, col_kv, gain_q, gain_kv, inv_freq,
                                                               rot_dims, tok_slot, tok_pos, block_table, max_blocks, (float*)pool, q_rank, kv_rank,
                                                               rot_dim, page_size, eps)));
  return check_cuda(cudaGetLastError(), "hyb_latent_prepare");
}

int qs_hyb_latent_query(void* qa, const void* qlat, const void* q, int64_t q_stride, const float* inv_freq, int rot_dims, const int32_t* tok_pos,
                        int tokens_n, int heads, int dim, int kv_rank, int rot_dim, int dtype, void* stream) {
  QS_REQUIRE(qa && qlat && q && tok_pos, "hyb_latent_query: null tensor");
  QS_REQUIRE(rot_dims % 2 == 0 && rot_dims >= 0 && rot_dims <= rot_dim && (rot_dims == 0 || inv_freq), "hyb_latent_query: bad rotation");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(tokens_n, heads);
  QS_DT(dtype,
        (latent_query_kernel<__nv_bfloat16><<<grid, 64, 0, s>>>((__nv_bfloat16*)qa, (const __nv_bfloat16*)qlat, (const __nv_bfloat16*)q, q_stride, inv_freq,
                                                                 rot_dims, tok_pos, tokens_n, heads, dim, kv_rank, rot_dim)),
        (latent_query_kernel<float><<<grid, 64, 0, s>>>((float*)qa, (const float*)qlat, (const float*)q, q_stride, inv_freq, rot_dims, tok_pos, tokens_n,
                                                         heads, dim, kv_rank, rot_dim)));
  return check_cuda(cudaGetLastError(), "hyb_latent_query");
}

int qs_hyb_latent_attention(void* out, const void* qa, const void* pool, const int32_t* tok_slot, const int32_t* tok_pos, const int32_t* block_table,
                            int max_blocks, int tokens_n, int heads, int kv_rank, int rot_dim, float scale, int page_size, int chunk, int window,
                            int dtype, void* stream) {
  QS_REQUIRE(out && qa && pool && tok_slot && tok_pos && block_table, "hyb_latent_attention: null tensor");
  QS_REQUIRE(heads > 0 && kv_rank > 0 && kv_rank <= 32 * kLatMaxVC && rot_dim >= 0 && page_size > 0, "hyb_latent_attention: bad sizes (kv_rank <= 512)");
  QS_REQUIRE(chunk >= 0 && window >= 0, "hyb_latent_attention: negative chunk or window");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
#define QS_LAT(ST)                                                                                                                               \
  do {                                                                                                                                           \
    if (heads > 8) return launch_latent_attention<ST, 4>(out, qa, pool, tok_slot, tok_pos, block_table, max_blocks, tokens_n, heads, kv_rank, rot_dim, \
                                                         scale, page_size, chunk, window, s);                                                   \
    if (heads > 4) return launch_latent_attention<ST, 2>(out, qa, pool, tok_slot, tok_pos, block_table, max_blocks, tokens_n, heads, kv_rank, rot_dim, \
                                                         scale, page_size, chunk, window, s);                                                   \
    return launch_latent_attention<ST, 1>(out, qa, pool, tok_slot, tok_pos, block_table, max_blocks, tokens_n, heads, kv_rank, rot_dim, scale,   \
                                          page_size, chunk, window, s);                                                                         \
  } while (0)
  QS_DT(dtype, QS_LAT(__nv_bfloat16), QS_LAT(float));
#undef QS_LAT
  return qs::QS_OK;
}

int qs_hyb_latent_attention_fast_supported(int dtype, int heads, int kv_rank, int rot_dim) { return 0; }

int64_t qs_hyb_latent_attention_scratch_floats(int tokens, int heads, int kv_rank) { return 0; }

int qs_hyb_latent_attention_fast(void* out, const void* qa, const void* pool, const int32_t* tok_slot, const int32_t* tok_pos, const int32_t* block_table,
                                 int max_blocks, const int32_t* entry_start, const int32_t* entry_len, const int32_t* entry_slot,
                                 const int32_t* entry_pos0, int entries, int tokens_n, float* scratch, int heads, int kv_rank, int rot_dim, float scale,
                                 int page_size, int chunk, int window, int dtype, void* stream) {
  return set_error(qs::QS_ERR_INVALID, "hyb_latent_attention_fast: shape not supported (use qs_hyb_latent_attention)");
}

int qs_hyb_latent_gate_out(void* out, int64_t out_stride, const void* ov, const void* gate, int64_t gate_stride, int col_g, int tokens_n, int heads,
                           int vdim, int dtype, void* stream) {
  QS_REQUIRE(out && ov, "hyb_latent_gate_out: null tensor");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  QS_DT(dtype,
        (latent_gate_out_kernel<__nv_bfloat16><<<tokens_n, 128, 0, s>>>((__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)ov, (const __nv_bfloat16*)gate,
                                                                         gate_stride, col_g, tokens_n, heads, vdim)),
        (latent_gate_out_kernel<float><<<tokens_n, 128, 0, s>>>((float*)out, out_stride, (const float*)ov, (const float*)gate, gate_stride, col_g, tokens_n,
                                                                heads, vdim)));
  return check_cuda(cudaGetLastError(), "hyb_latent_gate_out");
}

}  // extern "C"
