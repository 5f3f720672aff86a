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
// Rotation: layout 1 ("half") pairs entry i < dims/2 with entry i + dims/2, layout 0 ("interleaved") pairs entries (2i, 2i + 1); angle =
// position * inv_freq[i], cos and sin times `amp`; entries from `dims` on pass.  Q == 0: there is no query latent (cq is not written).
// ---------------------------------------------------------------------------------------------------------------------------------
template <typename ST>
__global__ void __launch_bounds__(128) latent_prepare_kernel(ST* __restrict__ cq, const ST* __restrict__ proj, long long stride, int col_q, int col_kv,
                                                             const float* __restrict__ gain_q, const float* __restrict__ gain_kv,
                                                             const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ tok_slot,
                                                             const int* __restrict__ tok_pos, const int* __restrict__ block_table, int max_blocks,
                                                             ST* __restrict__ pool, int Q, int K, int R, int page, float eps, int rot_layout,
                                                             float amp) {
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
  const float rq = Q > 0 ? 1.f / sqrtf(sq / (float)Q + eps) : 0.f, rk = 1.f / sqrtf(sk / (float)K + eps);
  for (int i = tid; i < Q; i += blockDim.x) stf(cq + (size_t)t * Q + i, ldf(row + col_q + i) * rq * gain_q[i]);
  const int pg = block_table[(size_t)tok_slot[t] * max_blocks + pos / page];
  ST* cell = pool + ((size_t)pg * page + pos % page) * (size_t)(K + R);
  for (int i = tid; i < K; i += blockDim.x) stf(cell + i, ldf(row + col_kv + i) * rk * gain_kv[i]);
  const ST* kr = row + col_kv + K;
  const int half = rot_dims >> 1;
  for (int i = tid; i < R; i += blockDim.x) {
    float v = ldf(kr + i);
    if (i < rot_dims) {
      const bool first = rot_layout == 0 ? (i & 1) == 0 : i < half;
      const int p = rot_layout == 0 ? i >> 1 : (first ? i : i - half);
      float s, c;
      sincosf((float)pos * inv_freq[p], &s, &c);
      const float a = ldf(kr + (rot_layout == 0 ? 2 * p : p)), b = ldf(kr + (rot_layout == 0 ? 2 * p + 1 : p + half));
      v = (first ? a * c - b * s : b * c + a * s) * amp;
    }
    stf(cell + K + i, v);
  }
}

// query rows of K + R numbers: qa[t][h] = [qlat[h][t][0:K] | rotate(q[t][h][D : D + R])] (qa may be null).  rotate_back: the rotated part
// also replaces q's own (the per-head keys of a prompt portion are scored against q as it lies).  One block per (token, head); a thread
// takes both entries of a rotated pair.
template <typename ST>
__global__ void __launch_bounds__(64) latent_query_kernel(ST* __restrict__ qa, const ST* __restrict__ qlat, ST* __restrict__ q, long long q_stride,
                                                          const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ tok_pos, int T, int H,
                                                          int D, int K, int R, int rotate_back, int rot_layout, float amp) {
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  ST* dst = qa != nullptr ? qa + ((size_t)t * H + h) * (size_t)(K + R) : nullptr;
  if (dst != nullptr) {
    const ST* src = qlat + ((size_t)h * T + t) * (size_t)K;
    for (int i = tid; i < K; i += blockDim.x) dst[i] = src[i];
  }
  ST* qr = q + (size_t)t * q_stride + (size_t)h * (D + R) + D;
  const int pos = tok_pos[t], half = rot_dims >> 1;
  for (int p = tid; p < half; p += blockDim.x) {
    float s, c;
    sincosf((float)pos * inv_freq[p], &s, &c);
    const int ia = rot_layout == 0 ? 2 * p : p, ib = rot_layout == 0 ? 2 * p + 1 : p + half;
    const float a = ldf(qr + ia), b = ldf(qr + ib);
    const float u = (a * c - b * s) * amp, v = (b * c + a * s) * amp;
    if (dst != nullptr) {
      stf(dst + K + ia, u);
      stf(dst + K + ib, v);
    }
    if (rotate_back) {
      stf(qr + ia, u);
      stf(qr + ib, v);
    }
  }
  if (dst != nullptr)
    for (int i = rot_dims + tid; i < R; i += blockDim.x) dst[K + i] = qr[i];
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
                                                               float scale, int page, int chunk, int window, const float* __restrict__ sinks) {
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
    // a sink is one more term exp(sink) of the denominator without a value: the running maximum and sum start from it
    const int hh = h0 + warp * HPW + u;
    const bool sunk = sinks != nullptr && hh < H;
    m_run[u] = sunk ? sinks[hh] : -INFINITY;
    l_run[u] = sunk ? 1.f : 0.f;
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
                            int max_blocks, int T, int H, int K, int R, float scale, int page, int chunk, int window, const float* sinks,
                            cudaStream_t s) {
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
                                                                                          block_table, max_blocks, T, H, K, R, scale, page, chunk, window, sinks);
  return check_cuda(cudaGetLastError(), "hyb_latent_attention");
}

// ---------------------------------------------------------------------------------------------------------------------------------
// Latent attention on the tensor cores (bfloat16 storage).  The 64 rows of a tile are (token, head) pairs of ONE sequence: RT = 64 / HB
// consecutive tokens x HB heads (row r: token r / HB, head r % HB).  All rows score the same cells, so a tile of 32 cells, streamed through
// the block table with cp.async into a double buffer, meets 64 queries; the cells' first K columns are also the values (no second copy).
// 8 warps: warp (rb, ch) owns rows [16 rb, 16 rb + 16) and the value columns [ch K/2, (ch + 1) K/2).  Both warps of a row block form the
// same scores S = Q C^T (mma.sync m16n8k16, bf16 operands, fp32 accumulation) and the same online softmax (base 2, fp32), so no exchange
// is needed; P V takes the fp32 weights as three bfloat16 terms (p = hi + mid + lo), i.e. at fp32 precision.
// LONG: blocks walk the tiles of entries of at least 16 tokens (tile_entry / tile_row0 name 64-token spans; a block takes RT tokens of one)
//       and write out [H][T][K] (bfloat16) directly.
// SHORT: one listed token per block row, the cells shared out over `splits` blocks (blockIdx.z); un-normalised partial sums, running
//       maximum and denominator go to `part` [n_short][H][splits][2 + K] fp32, latent_merge_kernel finishes.
// ---------------------------------------------------------------------------------------------------------------------------------
constexpr int kLtRows = 64, kLtPad = 8, kLtTokensPerSpan = 64;

// 8 warps = 2 column halves x (RB row blocks of 16 rows x KG = 4 / RB key groups).  With 64 live rows (RB = 4) every warp owns a row block and
// sees all cells of a tile.  A single token with few heads has 16 or 32 live rows (RB = 1, 2): the warps that would idle take a share of
// each tile's cells instead (16 cells per warp), keep their own running maximum / denominator / sums and are merged through shared memory
// at the end -- the per-warp chain of dependent MMAs per tile, which bounds a single token's step, is KG times shorter.
template <int RB> struct LtShape {
  static constexpr int KG = 4 / RB;            // key groups
  static constexpr int KT = KG == 4 ? 64 : 32;  // cells per tile
  static constexpr int KW = KT / KG;           // cells of a tile per warp: 32, 16, 16
  static constexpr int QR = 16 * RB;           // query rows held
};

template <int NVT, int RB, bool SHORT>  // K = 32 NVT: NVT value column blocks of 16 per warp
__global__ void __launch_bounds__(256, 1) latent_tile_kernel(
    __nv_bfloat16* __restrict__ out, float* __restrict__ part, const __nv_bfloat16* __restrict__ qa, const __nv_bfloat16* __restrict__ pool,
    const int* __restrict__ tile_entry, const int* __restrict__ tile_row0, const int* __restrict__ short_tokens, const int* __restrict__ tok_slot,
    const int* __restrict__ tok_pos, const int* __restrict__ entry_start, const int* __restrict__ entry_len, const int* __restrict__ entry_slot,
    const int* __restrict__ entry_pos0, const int* __restrict__ block_table, int max_blocks, int T, int H, int HB, int R, float scale, int page,
    int chunk, int window, int splits, const float* __restrict__ sinks) {
  extern __shared__ __align__(16) unsigned char smraw[];
  constexpr int K = 32 * NVT, KG = LtShape<RB>::KG, KT = LtShape<RB>::KT, KW = LtShape<RB>::KW, QR = LtShape<RB>::QR, TPR = 256 / KT;
  const int DK = K + R, DKP = (DK + 15) & ~15, SD = DKP + kLtPad;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw);  // [QR][SD]
  __nv_bfloat16* Ks = Qs + QR * SD;                             // [2][KT][SD]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, ch = warp >> 2, rb = (warp & 3) % RB, kg = (warp & 3) / RB;
  const int RT = QR / HB, h0 = blockIdx.y * HB;
  int tok0, n_tok, pos0, slot;
  if (SHORT) {
    tok0 = short_tokens[blockIdx.x];
    n_tok = 1;
    pos0 = tok_pos[tok0];
    slot = tok_slot[tok0];
  } else {
    const int per_span = kLtTokensPerSpan / RT;
    const int tile = blockIdx.x / per_span, sub = blockIdx.x - tile * per_span;
    const int e = tile_entry[tile], r0 = tile_row0[tile] + sub * RT;
    n_tok = min(RT, entry_len[e] - r0);
    if (n_tok <= 0) return;
    tok0 = entry_start[e] + r0;
    pos0 = entry_pos0[e] + r0;
    slot = entry_slot[e];
  }
  const int* bt = block_table + (size_t)slot * max_blocks;
  // queries: 16-byte chunks, zero rows for (token, head) pairs that do not exist, zero columns up to a multiple of 16
  const int dch = DK >> 3, sch = DKP >> 3;
  for (int c = tid; c < QR * sch; c += 256) {
    const int r = c / sch, cc = c - r * sch;
    const int tk = r / HB, hh = h0 + r % HB;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tk < n_tok && hh < H && cc < dch) v = *reinterpret_cast<const uint4*>(qa + ((size_t)(tok0 + tk) * H + hh) * DK + cc * 8);
    *reinterpret_cast<uint4*>(Qs + r * SD + cc * 8) = v;
  }
  const int last_pos = pos0 + n_tok - 1;
  int kt_lo = first_key(pos0, chunk, window) / KT, kt_hi = last_pos / KT + 1;  // tiles [kt_lo, kt_hi)
  if (SHORT) {
    const int per = (kt_hi - kt_lo + splits - 1) / splits;
    kt_lo += blockIdx.z * per;
    kt_hi = min(kt_hi, kt_lo + per);
  }
  const bool live = rb * 16 < n_tok * HB;  // a row block without any real (token, head) pair only helps to load
  const int qrow = rb * 16 + (lane >> 2);  // this thread's rows: qrow, qrow + 8
  const int qp[2] = {pos0 + min(qrow / HB, n_tok - 1), pos0 + min((qrow + 8) / HB, n_tok - 1)};
  const int fk[2] = {first_key(qp[0], chunk, window), first_key(qp[1], chunk, window)};
  const int warp_qp_min = pos0 + min(rb * 16 / HB, n_tok - 1);
  const float scale_log2 = scale * 1.4426950408889634f;
  float o[2 * NVT][4];
#pragma unroll
  for (int i = 0; i < 2 * NVT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  // TPR threads per cell row, alternating 16-byte chunks; the block-table lookup is made one tile ahead of its use
  auto cell_of = [&](int kt) -> long long {
    const int kp = kt * KT + tid / TPR;
    return kp <= last_pos ? (long long)bt[kp / page] * page + kp % page : -1;
  };
  auto load_tile = [&](int buf, long long cell) {
    __nv_bfloat16* Kd = Ks + ((size_t)buf * KT + tid / TPR) * SD;
    if (cell >= 0) {
      const __nv_bfloat16* src = pool + (size_t)cell * DK;
      for (int cc = tid % TPR; cc < sch; cc += TPR) {
        if (cc < dch) cp_async16(Kd + cc * 8, src + cc * 8);
        else *reinterpret_cast<uint4*>(Kd + cc * 8) = make_uint4(0, 0, 0, 0);
      }
    } else {
      for (int cc = tid % TPR; cc < sch; cc += TPR) *reinterpret_cast<uint4*>(Kd + cc * 8) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (kt_lo < kt_hi) load_tile(kt_lo & 1, cell_of(kt_lo));
  long long cell_next = kt_lo + 1 < kt_hi ? cell_of(kt_lo + 1) : -1;
  for (int kt = kt_lo; kt < kt_hi; ++kt) {
    if (kt + 1 < kt_hi) {
      load_tile((kt + 1) & 1, cell_next);
      if (kt + 2 < kt_hi) cell_next = cell_of(kt + 2);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    if (live) {
      const __nv_bfloat16* Kc = Ks + ((size_t)(kt & 1) * KT + kg * KW) * SD;  // this warp's cells of the tile
      float s[KW / 8][4];
#pragma unroll
      for (int i = 0; i < KW / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      for (int ks = 0; ks < DKP; ks += 16) {
        uint32_t a[4];
        ldsm_x4(a, Qs + (rb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * SD + ks + (lane >> 4) * 8);
#pragma unroll
        for (int np = 0; np < KW / 16; ++np) {
          uint32_t b[4];
          ldsm_x4(b, Kc + (np * 16 + (lane & 7) + (lane >> 4) * 8) * SD + ks + ((lane >> 3) & 1) * 8);
          mma_bf16(s[2 * np], a, b[0], b[1]);
          mma_bf16(s[2 * np + 1], a, b[2], b[3]);
        }
      }
      // scale, mask (rows of one warp belong to different tokens: each has its own last and first visible cell), online softmax
      float mx[2] = {-INFINITY, -INFINITY};
      const int k0 = kt * KT + kg * KW;
      const bool edge = k0 + KW - 1 > warp_qp_min || chunk > 0 || window > 0;
#pragma unroll
      for (int nt = 0; nt < KW / 8; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float v = s[nt][j] * scale_log2;
          if (edge) {
            const int kpos = k0 + nt * 8 + (lane & 3) * 2 + (j & 1);
            if (kpos > qp[j >> 1] || kpos < fk[j >> 1]) v = -INFINITY;
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
      for (int nt = 0; nt < KW / 8; ++nt)
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
      constexpr int NVG = NVT % 4 == 0 ? 4 : (NVT % 2 == 0 ? 2 : 1);
      const __nv_bfloat16* Vc = Kc + ch * (K / 2);  // the values: this warp's half of the cells' first K columns
#pragma unroll
      for (int kk = 0; kk < KW / 16; ++kk) {
        uint32_t a[3][4];
#pragma unroll
        for (int pt = 0; pt < 4; ++pt) {
          const int nt = 2 * kk + (pt >> 1), j0 = (pt & 1) * 2;
          float r0v = s[nt][j0], r1v = s[nt][j0 + 1];
#pragma unroll
          for (int sp = 0; sp < 3; ++sp) a[sp][pt] = split_bf16x2(r0v, r1v);
        }
#pragma unroll
        for (int nv0 = 0; nv0 < NVT; nv0 += NVG) {
          uint32_t b[NVG][4];
#pragma unroll
          for (int i = 0; i < NVG; ++i)
            ldsm_x4_trans(b[i], Vc + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * SD + (nv0 + i) * 16 + (lane >> 4) * 8);
#pragma unroll
          for (int sp = 0; sp < 3; ++sp)
#pragma unroll
            for (int i = 0; i < NVG; ++i) {
              mma_bf16(o[2 * (nv0 + i)], a[sp], b[i][0], b[i][1]);
              mma_bf16(o[2 * (nv0 + i) + 1], a[sp], b[i][2], b[i][3]);
            }
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
  if (KG > 1) {
    // the key groups of a row block meet in shared memory (the tiles are consumed): group 0 folds the others' (maximum, denominator, sums)
    constexpr int PER = 4 + 8 * NVT;  // floats per thread
    float* xs = reinterpret_cast<float*>(smraw);
    __syncthreads();  // a block without tiles comes here straight from writing the queries
    if (kg > 0) {
      float* d = xs + ((size_t)((ch * RB + rb) * (KG - 1) + kg - 1) * 32 + lane) * PER;
      d[0] = m_run[0]; d[1] = m_run[1]; d[2] = l_run[0]; d[3] = l_run[1];
#pragma unroll
      for (int i = 0; i < 2 * NVT; ++i) *reinterpret_cast<float4*>(d + 4 + 4 * i) = make_float4(o[i][0], o[i][1], o[i][2], o[i][3]);
    }
    __syncthreads();
    if (kg > 0) return;
#pragma unroll
    for (int g = 1; g < KG; ++g) {
      const float* d = xs + ((size_t)((ch * RB + rb) * (KG - 1) + g - 1) * 32 + lane) * PER;
      float fa[2], fb[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float mo = d[r], m_new = fmaxf(m_run[r], mo);
        fa[r] = m_new == -INFINITY ? 1.f : fast_exp2(m_run[r] - m_new);
        fb[r] = m_new == -INFINITY ? 0.f : fast_exp2(mo - m_new);
        m_run[r] = m_new;
        l_run[r] = l_run[r] * fa[r] + d[2 + r] * fb[r];
      }
#pragma unroll
      for (int i = 0; i < 2 * NVT; ++i) {
        const float4 v = *reinterpret_cast<const float4*>(d + 4 + 4 * i);
        o[i][0] = o[i][0] * fa[0] + v.x * fb[0]; o[i][1] = o[i][1] * fa[0] + v.y * fb[0];
        o[i][2] = o[i][2] * fa[1] + v.z * fb[1]; o[i][3] = o[i][3] * fa[1] + v.w * fb[1];
      }
    }
  }
  if (!live) return;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = qrow + r * 8, tk = row / HB, hh = h0 + row % HB;
    if (tk >= n_tok || hh >= H) continue;
    const int col0 = ch * (K / 2) + (lane & 3) * 2;
    if (SHORT) {
      float* dst = part + (((size_t)blockIdx.x * H + hh) * splits + blockIdx.z) * (size_t)(2 + K);
      if (ch == 0 && (lane & 3) == 0) {
        dst[0] = m_run[r];
        dst[1] = l_run[r];
      }
#pragma unroll
      for (int i = 0; i < 2 * NVT; ++i) *reinterpret_cast<float2*>(dst + 2 + col0 + i * 8) = make_float2(o[i][2 * r], o[i][2 * r + 1]);
    } else {
      // a sink joins the denominator as exp(sink) relative to the running maximum (base-2 domain); it has no value
      const float inv = 1.f / (l_run[r] + (sinks != nullptr ? fast_exp2(sinks[hh] * 1.4426950408889634f - m_run[r]) : 0.f));
      __nv_bfloat16* dst = out + ((size_t)hh * T + tok0 + tk) * (size_t)K + col0;
#pragma unroll
      for (int i = 0; i < 2 * NVT; ++i) *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
    }
  }
}

// out[h][t][:] = sum_z 2^(m_z - M) o_z / sum_z 2^(m_z - M) l_z over the key shares of a listed token.  One warp per (listed token, head).
__global__ void latent_merge_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ part, const int* __restrict__ short_tokens, int n_short,
                                    int T, int H, int K, int splits, const float* __restrict__ sinks) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= n_short * H) return;
  const int i = w / H, h = w - i * H;
  const float* p = part + (size_t)w * splits * (2 + K);
  const float sink2 = sinks != nullptr ? sinks[h] * 1.4426950408889634f : -INFINITY;  // the sink: a share of maximum sink, sum 1, no output
  float M = sink2;
  for (int z = 0; z < splits; ++z) M = fmaxf(M, p[(size_t)z * (2 + K)]);
  float L = sinks != nullptr ? fast_exp2(sink2 - M) : 0.f;
  for (int z = 0; z < splits; ++z) {
    const float m = p[(size_t)z * (2 + K)];
    if (m != -INFINITY) L += fast_exp2(m - M) * p[(size_t)z * (2 + K) + 1];
  }
  const float inv = 1.f / L;
  __nv_bfloat16* dst = out + ((size_t)h * T + short_tokens[i]) * (size_t)K;
  for (int c = lane; c < K; c += 32) {
    float a = 0.f;
    for (int z = 0; z < splits; ++z) {
      const float m = p[(size_t)z * (2 + K)];
      if (m != -INFINITY) a += fast_exp2(m - M) * p[(size_t)z * (2 + K) + 2 + c];
    }
    dst[c] = __float2bfloat16_rn(a * inv);
  }
}

// key shares of single tokens are chosen to give about one block per SM (148): a block of the widest latents takes most of an SM's shared
// memory, so a second wave of blocks would wait for the first (measured at 64 tokens x 1024 cells: 55 us against 63 us with twice the blocks)
constexpr int kLtTargetBlocks = 148;
constexpr int kLtMaxSplits = 16;

template <int RB> size_t latent_tile_smem(int K, int R) {
  const int sd = ((K + R + 15) & ~15) + kLtPad;
  const size_t tiles = (size_t)(LtShape<RB>::QR + 2 * LtShape<RB>::KT) * sd * sizeof(__nv_bfloat16);
  const size_t merge = (size_t)2 * RB * (LtShape<RB>::KG - 1) * 32 * (4 + K / 4) * sizeof(float);  // the key groups' meeting place
  return std::max(tiles, merge);
}

bool latent_fast_supported(int dtype, int heads, int kv_rank, int rot_dim) {
  if (dtype != QS_DTYPE_BF16 || heads < 1 || rot_dim < 0) return false;
  if (!(kv_rank == 32 || kv_rank == 64 || kv_rank == 128 || kv_rank == 256 || kv_rank == 512)) return false;
  const size_t most = std::max(latent_tile_smem<1>(kv_rank, rot_dim), std::max(latent_tile_smem<2>(kv_rank, rot_dim), latent_tile_smem<4>(kv_rank, rot_dim)));
  return (kv_rank + rot_dim) % 8 == 0 && most <= 200 * 1024;
}

int latent_head_block(int heads) { return heads <= 16 ? 16 : (heads <= 32 ? 32 : 64); }

int latent_splits(int n_short, int heads) {
  const int groups = (heads + latent_head_block(heads) - 1) / latent_head_block(heads);
  return std::max(1, std::min(kLtMaxSplits, kLtTargetBlocks / std::max(1, n_short * groups)));
}

template <int NVT, int RB>
int launch_latent_short(void* out, float* part, const void* qa, const void* pool, const int* short_tokens, int n_short, const int* tok_slot,
                        const int* tok_pos, const int* block_table, int max_blocks, int T, int H, int HB, int R, float scale, int page, int chunk,
                        int window, const float* sinks, cudaStream_t s) {
  const int K = 32 * NVT, groups = (H + HB - 1) / HB, splits = latent_splits(n_short, H);
  const size_t smem = latent_tile_smem<RB>(K, R);
  static bool attr_set[kMaxDevices] = {};
  if (!attr_set[device_ordinal()]) {
    if (int rc = check_cuda(cudaFuncSetAttribute(latent_tile_kernel<NVT, RB, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), "latent tiles smem")) return rc;
    attr_set[device_ordinal()] = true;
  }
  latent_tile_kernel<NVT, RB, true><<<dim3(n_short, groups, splits), 256, smem, s>>>(
      (__nv_bfloat16*)out, part, (const __nv_bfloat16*)qa, (const __nv_bfloat16*)pool, nullptr, nullptr, short_tokens, tok_slot, tok_pos, nullptr, nullptr,
      nullptr, nullptr, block_table, max_blocks, T, H, HB, R, scale, page, chunk, window, splits, nullptr);
  const int warps = n_short * H;
  latent_merge_kernel<<<(warps + 3) / 4, 128, 0, s>>>((__nv_bfloat16*)out, part, short_tokens, n_short, T, H, K, splits, sinks);
  return check_cuda(cudaGetLastError(), "hyb_latent_attention_fast single tokens");
}

template <int NVT>
int launch_latent_tiles(void* out, float* part, const void* qa, const void* pool, const int* tile_entry, const int* tile_row0, int n_tiles,
                        const int* short_tokens, int n_short, const int* tok_slot, const int* tok_pos, const int* entry_start, const int* entry_len,
                        const int* entry_slot, const int* entry_pos0, const int* block_table, int max_blocks, int T, int H, int R, float scale,
                        int page, int chunk, int window, const float* sinks, cudaStream_t s) {
  const int K = 32 * NVT, HB = latent_head_block(H), groups = (H + HB - 1) / HB;
  if (n_tiles > 0) {
    const size_t smem = latent_tile_smem<4>(K, R);
    static bool attr_set[kMaxDevices] = {};
    if (!attr_set[device_ordinal()]) {
      if (int rc = check_cuda(cudaFuncSetAttribute(latent_tile_kernel<NVT, 4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), "latent tiles smem")) return rc;
      attr_set[device_ordinal()] = true;
    }
    latent_tile_kernel<NVT, 4, false><<<dim3(n_tiles * (kLtTokensPerSpan / (kLtRows / HB)), groups), 256, smem, s>>>(
        (__nv_bfloat16*)out, nullptr, (const __nv_bfloat16*)qa, (const __nv_bfloat16*)pool, tile_entry, tile_row0, nullptr, tok_slot, tok_pos, entry_start,
        entry_len, entry_slot, entry_pos0, block_table, max_blocks, T, H, HB, R, scale, page, chunk, window, 1, sinks);
    if (int rc = check_cuda(cudaGetLastError(), "hyb_latent_attention_fast tiles")) return rc;
  }
  if (n_short > 0) {
    // a single token has HB live rows: 16 (one row block, four key groups), 32 (two and two) or 64 (four row blocks)
    if (HB == 16) return launch_latent_short<NVT, 1>(out, part, qa, pool, short_tokens, n_short, tok_slot, tok_pos, block_table, max_blocks, T, H, HB, R, scale, page, chunk, window, sinks, s);
    if (HB == 32) return launch_latent_short<NVT, 2>(out, part, qa, pool, short_tokens, n_short, tok_slot, tok_pos, block_table, max_blocks, T, H, HB, R, scale, page, chunk, window, sinks, s);
    return launch_latent_short<NVT, 4>(out, part, qa, pool, short_tokens, n_short, tok_slot, tok_pos, block_table, max_blocks, T, H, HB, R, scale, page, chunk, window, sinks, s);
  }
  return qs::QS_OK;
}

// out[t][h * Dv + j] = o * sigmoid(gate[t][col_g + h])   (gate == null: no gate; gate_wide: gate[t][col_g + h * Dv + j]).  o = ov[h][t][j] (head-major rows of the value
// up-projection), or, for tokens of entries of at least min_long tokens when `alt` is given, alt[t][h * Dv + j] (token-major rows of the
// per-head attention over a prompt portion).  One block per token.
template <typename ST>
__global__ void latent_gate_out_kernel(ST* __restrict__ out, long long out_stride, const ST* __restrict__ ov, const ST* __restrict__ alt,
                                       long long alt_stride, const int* __restrict__ tok_entry, const int* __restrict__ entry_len, int min_long,
                                       const ST* __restrict__ gate, long long gate_stride, int col_g, int T, int H, int Dv, int gate_wide) {
  const int t = blockIdx.x;
  const bool from_alt = alt != nullptr && entry_len[tok_entry[t]] >= min_long;
  for (int i = threadIdx.x; i < H * Dv; i += blockDim.x) {
    const int h = i / Dv, j = i - h * Dv;
    float v = from_alt ? ldf(alt + (size_t)t * alt_stride + i) : ldf(ov + ((size_t)h * T + t) * Dv + j);
    if (gate != nullptr) v *= 1.f / (1.f + expf(-ldf(gate + (size_t)t * gate_stride + col_g + (gate_wide ? i : h))));
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
                          int max_blocks, void* pool, int tokens_n, int q_rank, int kv_rank, int rot_dim, int page_size, float eps, int rot_layout,
                          float amplitude, int dtype, void* stream) {
  QS_REQUIRE(proj && gain_kv && tok_slot && tok_pos && block_table && pool && (q_rank == 0 || (cq && gain_q)), "hyb_latent_prepare: null tensor");
  QS_REQUIRE(q_rank >= 0 && kv_rank > 0 && rot_dim >= 0 && page_size > 0 && (rot_layout == 0 || rot_layout == 1), "hyb_latent_prepare: bad sizes");
  QS_REQUIRE(rot_dims % 2 == 0 && rot_dims >= 0 && rot_dims <= rot_dim && (rot_dims == 0 || inv_freq), "hyb_latent_prepare: bad rotation");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  QS_DT(dtype,
        (latent_prepare_kernel<__nv_bfloat16><<<tokens_n, 128, 0, s>>>((__nv_bfloat16*)cq, (const __nv_bfloat16*)proj, stride, col_q, col_kv, gain_q,
                                                                        gain_kv, inv_freq, rot_dims, tok_slot, tok_pos, block_table, max_blocks,
                                                                        (__nv_bfloat16*)pool, q_rank, kv_rank, rot_dim, page_size, eps, rot_layout,
                                                                        amplitude)),
        (latent_prepare_kernel<float><<<tokens_n, 128, 0, s>>>((float*)cq, (const float*)proj, stride, col_q, col_kv, gain_q, gain_kv, inv_freq,
                                                               rot_dims, tok_slot, tok_pos, block_table, max_blocks, (float*)pool, q_rank, kv_rank,
                                                               rot_dim, page_size, eps, rot_layout, amplitude)));
  return check_cuda(cudaGetLastError(), "hyb_latent_prepare");
}

int qs_hyb_latent_query(void* qa, const void* qlat, void* q, int64_t q_stride, const float* inv_freq, int rot_dims, const int32_t* tok_pos,
                        int tokens_n, int heads, int dim, int kv_rank, int rot_dim, int rotate_back, int rot_layout, float amplitude, int dtype,
                        void* stream) {
  QS_REQUIRE(rot_layout == 0 || rot_layout == 1, "hyb_latent_query: unknown rotary layout");
  QS_REQUIRE(q && tok_pos && (qa == nullptr || qlat != nullptr) && (qa != nullptr || rotate_back), "hyb_latent_query: null tensor");
  QS_REQUIRE(rot_dims % 2 == 0 && rot_dims >= 0 && rot_dims <= rot_dim && (rot_dims == 0 || inv_freq), "hyb_latent_query: bad rotation");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(tokens_n, heads);
  QS_DT(dtype,
        (latent_query_kernel<__nv_bfloat16><<<grid, 64, 0, s>>>((__nv_bfloat16*)qa, (const __nv_bfloat16*)qlat, (__nv_bfloat16*)q, q_stride, inv_freq, rot_dims,
                                                                 tok_pos, tokens_n, heads, dim, kv_rank, rot_dim, rotate_back, rot_layout, amplitude)),
        (latent_query_kernel<float><<<grid, 64, 0, s>>>((float*)qa, (const float*)qlat, (float*)q, q_stride, inv_freq, rot_dims, tok_pos, tokens_n, heads, dim,
                                                         kv_rank, rot_dim, rotate_back, rot_layout, amplitude)));
  return check_cuda(cudaGetLastError(), "hyb_latent_query");
}

int qs_hyb_latent_attention(void* out, const void* qa, const void* pool, const int32_t* tok_slot, const int32_t* tok_pos, const int32_t* block_table,
                            int max_blocks, int tokens_n, int heads, int kv_rank, int rot_dim, float scale, int page_size, int chunk, int window,
                            const float* sinks, int dtype, void* stream) {
  QS_REQUIRE(out && qa && pool && tok_slot && tok_pos && block_table, "hyb_latent_attention: null tensor");
  QS_REQUIRE(heads > 0 && kv_rank > 0 && kv_rank <= 32 * kLatMaxVC && rot_dim >= 0 && page_size > 0, "hyb_latent_attention: bad sizes (kv_rank <= 512)");
  QS_REQUIRE(chunk >= 0 && window >= 0, "hyb_latent_attention: negative chunk or window");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
#define QS_LAT(ST)                                                                                                                               \
  do {                                                                                                                                           \
    if (heads > 8) return launch_latent_attention<ST, 4>(out, qa, pool, tok_slot, tok_pos, block_table, max_blocks, tokens_n, heads, kv_rank, rot_dim, \
                                                         scale, page_size, chunk, window, sinks, s);                                            \
    if (heads > 4) return launch_latent_attention<ST, 2>(out, qa, pool, tok_slot, tok_pos, block_table, max_blocks, tokens_n, heads, kv_rank, rot_dim, \
                                                         scale, page_size, chunk, window, sinks, s);                                            \
    return launch_latent_attention<ST, 1>(out, qa, pool, tok_slot, tok_pos, block_table, max_blocks, tokens_n, heads, kv_rank, rot_dim, scale,   \
                                          page_size, chunk, window, sinks, s);                                                                  \
  } while (0)
  QS_DT(dtype, QS_LAT(__nv_bfloat16), QS_LAT(float));
#undef QS_LAT
  return qs::QS_OK;
}

int qs_hyb_latent_attention_fast_supported(int dtype, int heads, int kv_rank, int rot_dim) {
  return latent_fast_supported(dtype, heads, kv_rank, rot_dim) ? 1 : 0;
}

int64_t qs_hyb_latent_attention_scratch_floats(int tokens, int heads, int kv_rank) {
  // the key shares of single tokens: [tokens x shares][heads][2 + kv_rank]; tokens x shares never exceeds tokens + the target block count
  return ((int64_t)tokens + kLtTargetBlocks) * heads * (2 + kv_rank);
}

int qs_hyb_latent_attention_fast(void* out, const void* qa, const void* pool, const int32_t* tok_slot, const int32_t* tok_pos, const int32_t* block_table,
                                 int max_blocks, const int32_t* tile_entry, const int32_t* tile_row0, int n_tiles, const int32_t* short_tokens,
                                 int n_short, const int32_t* entry_start, const int32_t* entry_len, const int32_t* entry_slot,
                                 const int32_t* entry_pos0, int tokens_n, float* scratch, int heads, int kv_rank, int rot_dim, float scale,
                                 int page_size, int chunk, int window, const float* sinks, int dtype, void* stream) {
  QS_REQUIRE(out && qa && pool && tok_slot && tok_pos && block_table, "hyb_latent_attention_fast: null tensor");
  QS_REQUIRE(latent_fast_supported(dtype, heads, kv_rank, rot_dim), "hyb_latent_attention_fast: shape not supported (use qs_hyb_latent_attention)");
  QS_REQUIRE(chunk >= 0 && window >= 0 && page_size > 0, "hyb_latent_attention_fast: bad mask or page size");
  QS_REQUIRE(n_tiles == 0 || (tile_entry && tile_row0 && entry_start && entry_len && entry_slot && entry_pos0), "hyb_latent_attention_fast: null tile table");
  QS_REQUIRE(n_short == 0 || (short_tokens && scratch), "hyb_latent_attention_fast: null token list");
  cudaStream_t s = (cudaStream_t)stream;
#define QS_LT(NVT)                                                                                                                              \
  return launch_latent_tiles<NVT>(out, scratch, qa, pool, tile_entry, tile_row0, n_tiles, short_tokens, n_short, tok_slot, tok_pos, entry_start, \
                                  entry_len, entry_slot, entry_pos0, block_table, max_blocks, tokens_n, heads, rot_dim, scale, page_size, chunk, window, sinks, s)
  switch (kv_rank / 32) {
    case 1: QS_LT(1);
    case 2: QS_LT(2);
    case 4: QS_LT(4);
    case 8: QS_LT(8);
    default: QS_LT(16);
  }
#undef QS_LT
}

int qs_hyb_latent_gate_out(void* out, int64_t out_stride, const void* ov, const void* alt, int64_t alt_stride, const int32_t* tok_entry,
                           const int32_t* entry_len, int min_long, const void* gate, int64_t gate_stride, int col_g, int tokens_n, int heads, int vdim,
                           int gate_wide, int dtype, void* stream) {
  QS_REQUIRE(out && (ov || alt), "hyb_latent_gate_out: null tensor");
  QS_REQUIRE(alt == nullptr || (tok_entry && entry_len), "hyb_latent_gate_out: the second source needs the entry tables");
  QS_REQUIRE(ov != nullptr || min_long <= 1, "hyb_latent_gate_out: without head-major rows every token must come from the second source");
  if (tokens_n == 0) return qs::QS_OK;
  cudaStream_t s = (cudaStream_t)stream;
  QS_DT(dtype,
        (latent_gate_out_kernel<__nv_bfloat16><<<tokens_n, 128, 0, s>>>((__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)ov, (const __nv_bfloat16*)alt,
                                                                         alt_stride, tok_entry, entry_len, min_long, (const __nv_bfloat16*)gate, gate_stride,
                                                                         col_g, tokens_n, heads, vdim, gate_wide)),
        (latent_gate_out_kernel<float><<<tokens_n, 128, 0, s>>>((float*)out, out_stride, (const float*)ov, (const float*)alt, alt_stride, tok_entry, entry_len,
                                                                min_long, (const float*)gate, gate_stride, col_g, tokens_n, heads, vdim, gate_wide)));
  return check_cuda(cudaGetLastError(), "hyb_latent_gate_out");
}

}  // extern "C"
