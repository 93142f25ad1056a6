// Dense GQA decode, the HBM-bound path: K and V tiles stream through a TMA ring into shared memory
// and are consumed by mma.sync with the query heads of one KV head as the M dimension.
//
// One CTA per (KV split, KV head, batch row): warp 0 is the TMA producer (64-token K and V
// tiles, 32 KB per stage, 3 stages, two CTAs per SM), warps 1-4 each own 16 tokens of every tile:
//   S[16 heads x 16 tokens] = Q . K^T   (A = Q fragments held in registers, B = ldmatrix of K)
//   online softmax per head row in the log2 domain (row max / sum over the 4 lanes of a row)
//   O[16 heads x 128 dims] += P . V     (A = P from the S accumulators, B = ldmatrix.trans of V)
// G <= 16 query heads per KV head are padded to the 16 rows of the MMA; the padding rows cost
// tensor throughput the path does not need.  At the end the four warps' (m, l, O) are merged
// through shared memory into one normalised partial + log-sum-exp per split; merge_kernel then
// combines the splits.  All mbarrier waits are bounded.
#include "sm100_common.cuh"

namespace xkv {
using namespace sm100;
namespace {

constexpr int D = 128;            // head dim of K and V
constexpr int TILE = 64;          // tokens per stage
constexpr int STAGES = 3;
constexpr int KV_BYTES = TILE * D * 2;        // 16 KB per tile of K or V
constexpr int STAGE_BYTES = 2 * KV_BYTES;     // K + V
constexpr int NWARPS = 4;                     // compute warps
constexpr int NTHREADS = 32 * (NWARPS + 1);
constexpr int OFF_BAR = STAGES * STAGE_BYTES;             // 98304
constexpr int OFF_MISC = OFF_BAR + 2 * STAGES * 8;
constexpr int SMEM_USED = OFF_MISC + 16;
constexpr int SMEM_BYTES = SMEM_USED + 1024;
// the epilogue reuses the ring: 4 warps x 16 rows x (128 dims + m + l) fp32
static_assert(NWARPS * 16 * (D + 2) * 4 <= STAGES * STAGE_BYTES, "merge scratch must fit in the ring");

struct Args {
  int batch, kv_len, num_heads, num_kv_heads, group;   // group = heads per KV head (<= 16)
  int num_splits, tiles_per_row;
  float scale_log2;          // sm_scale * log2(e)
  const void* q;
  int64_t q_sb, q_sh;
  float* partial_o;          // [batch][H][splits][128]
  float* lse;                // [batch][H][splits]
  int* status;
  float* logits;             // logits-only mode: fp32 sm_scale * q.k at [b * lg_sb + h * lg_sh + token]
  int64_t lg_sb, lg_sh;
  float sm_scale;
  const int32_t* kv_lens;    // per-row lengths (ragged batches) or NULL
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi, __nv_bfloat16) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi, __half) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack2(uint32_t u, __nv_bfloat16) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}
__device__ __forceinline__ float2 unpack2(uint32_t u, __half) {
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}

// MODE 0: the whole decode.  MODE 1 (LO): logits only (first pass of a two-pass decode): K is streamed,
// V is not, no softmax / P.V.  MODE 2 (FL): the scores come as fp32 logits from a first pass (keys that
// are not dense: factorized without RoPE); only V is streamed.
template <typename T, int MODE>
__global__ void __launch_bounds__(NTHREADS, 2)
dense_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const Args a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  constexpr bool LO = MODE == 1, FL = MODE == 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int row_len = a.kv_lens ? min(max(a.kv_lens[b], 0), a.kv_len) : a.kv_len;   // this row's length
  const int row_tiles = a.kv_lens ? (row_len + TILE - 1) / TILE : a.tiles_per_row;
  const int tile_begin = (int)(((int64_t)split * row_tiles) / a.num_splits);
  const int tile_end = (int)(((int64_t)(split + 1) * row_tiles) / a.num_splits);
  const uint32_t bar0 = base + OFF_BAR;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (STAGES + s); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_MISC);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), NWARPS); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  const int G = a.group;
  const int g = lane >> 2, t = lane & 3;
  // per-warp running state, rows g and g + 8 of the 16 padded head rows
  float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F};
  float l_run[2] = {0.f, 0.f};
  float oacc[16][4];
#pragma unroll
  for (int n = 0; n < 16; ++n) { oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f; }

  if (warp == 0) {
    // =========================== TMA producer =================================================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = tile_begin; tile < tile_end; ++tile) {
        if (!mbar_wait(bar_empty(stage), phase ^ 1u, abort_flag)) {
          report(a.status, XKV_ERR_TIMEOUT, 0, tile, kvh, b);
          break;
        }
        mbar_expect_tx(bar_full(stage), (LO || FL) ? KV_BYTES : STAGE_BYTES);
        const uint32_t sk = base + stage * STAGE_BYTES;
        if (!FL) {
          tma_load_4d(sk, &tmK, 0, kvh, tile * TILE, b, bar_full(stage));
          tma_load_4d(sk + KV_BYTES / 2, &tmK, 64, kvh, tile * TILE, b, bar_full(stage));
        }
        if (!LO) {
          tma_load_4d(sk + KV_BYTES, &tmV, 0, kvh, tile * TILE, b, bar_full(stage));
          tma_load_4d(sk + KV_BYTES + KV_BYTES / 2, &tmV, 64, kvh, tile * TILE, b, bar_full(stage));
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    // =========================== compute warps ================================================
    const int cw = warp - 1;                 // tokens cw*16 .. cw*16+15 of every tile
    // Q fragments: A operand (16 heads x 16 dims per k-step), rows >= G are zero
    uint32_t qf[8][4];
    if (!FL) {
      const T* qg = static_cast<const T*>(a.q) + (int64_t)b * a.q_sb + (int64_t)(kvh * G) * a.q_sh;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int row = g + (r & 1) * 8, col = ks * 16 + 2 * t + (r >> 1) * 8;
          qf[ks][r] = row < G ? *reinterpret_cast<const uint32_t*>(qg + (int64_t)row * a.q_sh + col) : 0u;
        }
      }
    }
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    // FL: this warp's 16 tokens x the 16 padded head rows of a tile, in the accumulator layout of S, loaded one
    // tile ahead (the loads of tile + 1 are in flight while tile is worked on; token pairs as 8-byte loads when the
    // rows allow it)
    float sc_next[2][4];
    const bool lg_pairs = FL && a.lg_sb % 2 == 0 && a.lg_sh % 2 == 0 && (reinterpret_cast<uintptr_t>(a.logits) & 7u) == 0;
    auto load_logits = [&](int tile, float (&dst)[2][4]) {
      const int tokb = tile * TILE + cw * 16 + 2 * t;
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int jr = 0; jr < 2; ++jr) {
          const int row = g + jr * 8, tok = tokb + n * 8;
          const float* src = a.logits + (int64_t)b * a.lg_sb + (int64_t)(kvh * G + row) * a.lg_sh + tok;
          if (row < G && lg_pairs && tok + 1 < row_len) {
            const float2 v = __ldg(reinterpret_cast<const float2*>(src));
            dst[n][2 * jr] = v.x;
            dst[n][2 * jr + 1] = v.y;
          } else {
            dst[n][2 * jr] = (row < G && tok < row_len) ? __ldg(src) : 0.f;
            dst[n][2 * jr + 1] = (row < G && tok + 1 < row_len) ? __ldg(src + 1) : 0.f;
          }
        }
    };
    if (FL && tile_begin < tile_end) load_logits(tile_begin, sc_next);
    for (int tile = tile_begin; tile < tile_end && alive; ++tile) {
      float sc[2][4];
      if (FL) {
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int j = 0; j < 4; ++j) sc[n][j] = sc_next[n][j];
        if (tile + 1 < tile_end) load_logits(tile + 1, sc_next);
      }
      bool ok = mbar_wait(bar_full(stage), phase, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) report(a.status, XKV_ERR_TIMEOUT, 1, tile, kvh, b);
        alive = false;
        break;
      }
      const uint32_t sk = base + stage * STAGE_BYTES, sv = sk + KV_BYTES;
      // ---- S = Q . K^T for this warp's 16 tokens: two 8-token n-tiles ---------------------------
      if (!FL) {
#pragma unroll
        for (int n = 0; n < 2; ++n) { sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f; }
      }
      if (!FL) {
        // ldmatrix (non-transposed): lanes 0-7 / 8-15 address tokens of n-tile 0 (dims k0.., k0+8..),
        // lanes 16-23 / 24-31 the tokens of n-tile 1
        const int mi = lane >> 3, r = lane & 7;
        const int token = cw * 16 + (mi >> 1) * 8 + r;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const int dim = ks * 16 + (mi & 1) * 8;
          const uint32_t ka = sk + (dim >> 6) * (KV_BYTES / 2) + token * 128 + ((((dim & 63) >> 3) ^ (token & 7)) << 4);
          uint32_t kb[4];
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(kb[0]), "=r"(kb[1]), "=r"(kb[2]), "=r"(kb[3])
                       : "r"(ka));
          TypeTraits<T>::mma(sc[0], qf[ks], kb[0], kb[1]);
          TypeTraits<T>::mma(sc[1], qf[ks], kb[2], kb[3]);
        }
      }
      const int tok0 = tile * TILE + cw * 16 + 2 * t;
      if (LO) {
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          const int row = g + rr * 8;
          if (row < G) {
            float* lg = a.logits + (int64_t)b * a.lg_sb + (int64_t)(kvh * G + row) * a.lg_sh;
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int tok = tok0 + n * 8 + e;
                if (tok < row_len) lg[tok] = sc[n][rr * 2 + e] * a.sm_scale;
              }
          }
        }
        __syncwarp();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (lane == 0) mbar_arrive(bar_empty(stage));
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        continue;
      }
      // ---- online softmax, rows g (c0,c1) and g+8 (c2,c3) -------------------------------------------
      float p[2][4];
      float alpha[2];
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        float v[4];
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int tok = tok0 + n * 8 + e;
            v[n * 2 + e] = tok < row_len ? sc[n][rr * 2 + e] * (FL ? 1.4426950408889634f : a.scale_log2) : -CUDART_INF_F;
          }
        float mx = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[rr], mx);
        const float m_use = m_new == -CUDART_INF_F ? 0.f : m_new;
        alpha[rr] = exp2f(m_run[rr] - m_use);
        m_run[rr] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          // round to the working dtype first: the row sum must match what P.V multiplies with
          const uint32_t pk = pack2(exp2f(v[i] - m_use), 0.f, T());
          p[rr][i] = unpack2(pk, T()).x;
          sum += p[rr][i];
        }
        l_run[rr] = l_run[rr] * alpha[rr] + sum;
      }
      // P as the A operand (16 heads x 16 tokens): n-tile 0 -> k 0..7, n-tile 1 -> k 8..15
      uint32_t pf[4];
      pf[0] = pack2(p[0][0], p[0][1], T());
      pf[1] = pack2(p[1][0], p[1][1], T());
      pf[2] = pack2(p[0][2], p[0][3], T());
      pf[3] = pack2(p[1][2], p[1][3], T());
      // ---- O = O * alpha + P . V ---------------------------------------------------------------------
      if (a.kv_lens != nullptr && (tile + 1) * TILE > row_len) {
        // Ragged batch, last tile of the row: value rows past the row's own length are outside the
        // call (they may hold anything, NaN included, and 0 * NaN is NaN).  Each warp zeroes those
        // among its own 16 tokens before reading them.
        const int first = max(row_len - tile * TILE, cw * 16);
        for (int idx = lane; idx < (cw * 16 + 16 - first) * 16; idx += 32) {
          const int token = first + (idx >> 4), ch = idx & 15;
          const uint32_t za = sv + (ch >> 3) * (KV_BYTES / 2) + token * 128 + ((ch & 7) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(za), "r"(0u) : "memory");
        }
        __syncwarp();
      }
      {
        const int mi = lane >> 3, r = lane & 7;
        const int token = cw * 16 + (mi & 1) * 8 + r;       // matrices 0/1: tokens 0-7 / 8-15 of dims n0..
#pragma unroll
        for (int np = 0; np < 8; ++np) {                    // pairs of 8-dim n-tiles
          const int dim = np * 16 + (mi >> 1) * 8;
          const uint32_t va = sv + (dim >> 6) * (KV_BYTES / 2) + token * 128 + ((((dim & 63) >> 3) ^ (token & 7)) << 4);
          uint32_t vb[4];
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(vb[0]), "=r"(vb[1]), "=r"(vb[2]), "=r"(vb[3])
                       : "r"(va));
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2) {
            float (&o)[4] = oacc[np * 2 + h2];
            o[0] *= alpha[0]; o[1] *= alpha[0]; o[2] *= alpha[1]; o[3] *= alpha[1];
            TypeTraits<T>::mma(o, pf, vb[h2 * 2], vb[h2 * 2 + 1]);
          }
        }
      }
      // release the stage: generic-proxy reads above, async-proxy refill next
      __syncwarp();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      if (lane == 0) mbar_arrive(bar_empty(stage));
      if (++stage == STAGES) { stage = 0; phase ^= 1u; }
    }
  }

  // =========================== merge the four warps ==============================================
  __syncthreads();   // every issued tile has been consumed (or the CTA is aborting): the ring is free
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    return;
  }
  if (LO) return;
  float* scratch = reinterpret_cast<float*>(sm);            // [warp][row 16][D + 2]
  if (warp >= 1) {
    const int cw = warp - 1;
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      float l = l_run[rr];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      float* rowp = scratch + (cw * 16 + g + rr * 8) * (D + 2);
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        rowp[n * 8 + 2 * t] = oacc[n][rr * 2];
        rowp[n * 8 + 2 * t + 1] = oacc[n][rr * 2 + 1];
      }
      if (t == 0) { rowp[D] = m_run[rr]; rowp[D + 1] = l; }
    }
  }
  __syncthreads();
  const int H = a.num_heads;
  for (int idx = threadIdx.x; idx < G * D; idx += NTHREADS) {
    const int row = idx / D, d = idx - row * D;
    float M = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, scratch[(w * 16 + row) * (D + 2) + D]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) {
      const float* rp = scratch + (w * 16 + row) * (D + 2);
      const float wgt = rp[D] == -CUDART_INF_F ? 0.f : exp2f(rp[D] - M);
      num = fmaf(wgt, rp[d], num);
      den = fmaf(wgt, rp[D + 1], den);
    }
    const int h = kvh * G + row;
    a.partial_o[(((int64_t)b * H + h) * a.num_splits + split) * D + d] = den > 0.f ? num / den : 0.f;
    if (d == 0)
      a.lse[((int64_t)b * H + h) * a.num_splits + split] =
          den > 0.f ? (M + log2f(den)) * 0.6931471805599453f : -CUDART_INF_F;
  }
}

template <typename T, int MODE>
int launch(const CUtensorMap& tK, const CUtensorMap& tV, const Args& a, cudaStream_t st) {
  auto kern = dense_tc_kernel<T, MODE>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) {
    cudaGetLastError();
    return XKV_ERR_LAUNCH;
  }
  kern<<<dim3(a.num_splits, a.num_kv_heads, a.batch), NTHREADS, SMEM_BYTES, st>>>(tK, tV, a);
  return cudaGetLastError() == cudaSuccess ? XKV_OK : XKV_ERR_LAUNCH;
}

bool encode_kv(CUtensorMap* m, int dtype, const void* ptr, int kvh, int L, int batch, int64_t sh, int64_t sl, int64_t sb) {
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)kvh, (cuuint64_t)L, (cuuint64_t)batch};
  const int64_t sbb = batch > 1 ? sb : (int64_t)L * kvh * D * 4;
  const cuuint64_t strides[3] = {(cuuint64_t)(kvh > 1 ? sh : D) * 2, (cuuint64_t)sl * 2, (cuuint64_t)sbb * 2};
  const cuuint32_t box[4] = {64, 1, TILE, 1};
  return encode_tiled_16bit(m, dtype, 4, ptr, dims, strides, box);
}

}  // namespace

static bool keys_ok(const xkv_decode_params& p) {
  if (p.score_mode != XKV_SCORE_DENSE) return false;
  if (p.dtype != XKV_BF16 && p.dtype != XKV_F16) return false;
  if (p.head_dim != D || p.tail_dim != 0 || p.logit_cap > 0.f) return false;
  if (p.mask) return false;   // additive masks run on the portable kernels
  if (p.num_heads / p.num_kv_heads > 16) return false;
  if (!aligned16(p.k) || (reinterpret_cast<uintptr_t>(p.q) & 3u)) return false;
  if (!stride_ok(p.k_sl) || (p.num_kv_heads > 1 && !stride_ok(p.k_sh)) || (p.batch > 1 && !stride_ok(p.k_sb))) return false;
  if (p.q_sh % 2 != 0 || p.q_sb % 2 != 0) return false;
  return true;
}

bool dense_tc_supported(const xkv_decode_params& p) {
  if (!keys_ok(p) || p.value_mode != XKV_VALUE_DENSE || (p.flags & XKV_FLAG_LOGITS_ONLY)) return false;
  if (p.value_dim != D || !aligned16(p.v) || !stride_ok(p.v_sl)) return false;
  if (p.num_kv_heads > 1 && !stride_ok(p.v_sh)) return false;
  if (p.batch > 1 && !stride_ok(p.v_sb)) return false;
  return true;
}

// Second pass for keys that are not dense: softmax over fp32 logits and P.V with dense values.
bool dense_tc_values_supported(const xkv_decode_params& p) {
  if (p.value_mode != XKV_VALUE_DENSE || (p.flags & (XKV_FLAG_LOGITS_ONLY | XKV_FLAG_FORCE_GENERIC))) return false;
  if (p.dtype != XKV_BF16 && p.dtype != XKV_F16) return false;
  if (p.logit_cap > 0.f || p.mask || p.num_heads / p.num_kv_heads > 16) return false;
  if (p.value_dim != D || !aligned16(p.v) || !stride_ok(p.v_sl)) return false;
  if (p.num_kv_heads > 1 && !stride_ok(p.v_sh)) return false;
  if (p.batch > 1 && !stride_ok(p.v_sb)) return false;
  return true;
}

int dense_tc_values_from_logits(const xkv_decode_params& p, const DenseTcPlan& pl, const LogitsSink& logits, void* ws,
                                int* status, cudaStream_t st) {
  char* w = static_cast<char*>(ws);
  CUtensorMap tV;
  if (!encode_kv(&tV, p.dtype, p.v, p.num_kv_heads, p.kv_len, p.batch, p.v_sh, p.v_sl, p.v_sb)) return XKV_ERR_NO_DEVICE;
  Args a;
  a.batch = p.batch; a.kv_len = p.kv_len; a.num_heads = p.num_heads; a.num_kv_heads = p.num_kv_heads;
  a.group = p.num_heads / p.num_kv_heads;
  a.num_splits = pl.num_splits; a.tiles_per_row = pl.tiles;
  a.scale_log2 = 1.4426950408889634f;
  a.q = nullptr; a.q_sb = a.q_sh = 0;
  a.partial_o = reinterpret_cast<float*>(w + pl.off_partial);
  a.lse = reinterpret_cast<float*>(w + pl.off_lse);
  a.status = status;
  a.logits = logits.ptr; a.lg_sb = logits.sb; a.lg_sh = logits.sh; a.sm_scale = 1.f;
  a.kv_lens = p.kv_lens;
  const int rc = p.dtype == XKV_BF16 ? launch<__nv_bfloat16, 2>(tV, tV, a, st) : launch<__half, 2>(tV, tV, a, st);
  if (rc != XKV_OK) return rc;
  return launch_merge(a.partial_o, a.lse, p.out, p.dtype, p.batch, p.num_heads, pl.num_splits, D, D, nullptr, 1, 0, 0,
                      0, 0, p.o_sb, p.o_sh, st, 0, 0, p.lse_out, p.lse_sb);
}

// First pass of the two-pass decode: fp32 logits of dense keys.
bool dense_tc_logits_supported(const xkv_decode_params& p) {
  return keys_ok(p) && !(p.flags & XKV_FLAG_FORCE_GENERIC);
}

bool dense_tc_plan(const xkv_decode_params& p, DenseTcPlan* pl) {
  const int tiles = ceil_div(p.kv_len, TILE);
  const int slots = 2 * device_sm_count();            // two CTAs per SM
  const int rows = p.batch * p.num_kv_heads;
  int best_s = 1;
  int64_t best_cost = -1;
  const int max_s = tiles < 128 ? tiles : 128;
  for (int s = 1; s <= max_s; ++s) {
    const int64_t waves = ceil_div(rows * s, slots);
    const int64_t cost = waves * (ceil_div(tiles, s) + 2);   // + a couple of tiles of fixed cost per CTA
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_s = s; }
  }
  pl->num_splits = best_s;
  pl->tiles = tiles;
  size_t off = 256;
  pl->off_partial = off;
  off += align_up((size_t)p.batch * p.num_heads * best_s * D * sizeof(float), 256);
  pl->off_lse = off;
  off += align_up((size_t)p.batch * p.num_heads * best_s * sizeof(float), 256);
  pl->total_bytes = off;
  return true;
}

int dense_tc_decode(const xkv_decode_params& p, const DenseTcPlan& pl, void* ws, cudaStream_t st,
                    const LogitsSink* sink) {
  char* w = static_cast<char*>(ws);
  CUtensorMap tK, tV;
  if (!encode_kv(&tK, p.dtype, p.k, p.num_kv_heads, p.kv_len, p.batch, p.k_sh, p.k_sl, p.k_sb)) return XKV_ERR_NO_DEVICE;
  if (sink) {
    tV = tK;
  } else if (!encode_kv(&tV, p.dtype, p.v, p.num_kv_heads, p.kv_len, p.batch, p.v_sh, p.v_sl, p.v_sb)) {
    return XKV_ERR_NO_DEVICE;
  }
  int* status = reinterpret_cast<int*>(w);
  clear_status_kernel<<<1, 64, 0, st>>>(status);
  Args a;
  a.batch = p.batch; a.kv_len = p.kv_len; a.num_heads = p.num_heads; a.num_kv_heads = p.num_kv_heads;
  a.group = p.num_heads / p.num_kv_heads;
  a.num_splits = pl.num_splits; a.tiles_per_row = pl.tiles;
  a.scale_log2 = p.sm_scale * 1.4426950408889634f;
  a.q = p.q; a.q_sb = p.q_sb; a.q_sh = p.q_sh;
  a.partial_o = reinterpret_cast<float*>(w + pl.off_partial);
  a.lse = reinterpret_cast<float*>(w + pl.off_lse);
  a.status = status;
  a.logits = nullptr; a.lg_sb = a.lg_sh = 0; a.sm_scale = p.sm_scale;
  a.kv_lens = p.kv_lens;
  if (sink) {
    a.logits = sink->ptr; a.lg_sb = sink->sb; a.lg_sh = sink->sh;
    return p.dtype == XKV_BF16 ? launch<__nv_bfloat16, 1>(tK, tV, a, st) : launch<__half, 1>(tK, tV, a, st);
  }
  const int rc = p.dtype == XKV_BF16 ? launch<__nv_bfloat16, 0>(tK, tV, a, st) : launch<__half, 0>(tK, tV, a, st);
  if (rc != XKV_OK) return rc;
  return launch_merge(a.partial_o, a.lse, p.out, p.dtype, p.batch, p.num_heads, pl.num_splits, D, D, nullptr, 1, 0, 0,
                      0, 0, p.o_sb, p.o_sh, st, 0, 0, p.lse_out, p.lse_sb);
}

}  // namespace xkv
