// Decode attention over a shared latent stream (absorbed factorized K / V, MLA): every query head
// scores the same rows A[b, l, :] (+ a decoupled RoPE tail) and accumulates the same value rows, so
// the heads are the M dimension of the MMAs and the latent is streamed exactly once per head block.
//
// One CTA per (KV split, block of HB heads, batch row), eight warps.  A TMA ring holds 32-token
// tiles of the key latent (64-column, 128-byte-swizzled blocks), the tail and, unless the values
// alias the key latent (MLA), the value latent; the last warp to finish a stage refills it.  Per tile:
//   S[HB x 32] = Q_eff . K_tile^T   split into (16 heads x 8 tokens) units over the warps, Q_eff
//                                   (bf16, HB x Dk) resident in shared memory, ldmatrix operands
//   tile max per head through shared memory, P = exp2(S - m) -> shared memory (bf16)
//   O[HB x Rv] += P . V_tile        each warp owns Rv/8 value columns for all HB heads
// Row sums are kept per thread and reduced once at the end.  Output: normalised partial in latent
// space + log-sum-exp per split; merge_kernel combines the splits and applies B_v / W_uv.
#include "sm100_common.cuh"

namespace xkv {
using namespace sm100;
namespace {

constexpr int TILE = 32;                // tokens per stage
constexpr int NCW = 8;                  // compute warps
constexpr int NTHREADS = 32 * NCW;      // no producer warp: the last warp to finish a stage refills it
constexpr int MAX_SMEM = 232448 - 1024;

struct Args {
  int batch, kv_len, num_heads;
  int dk, rk, rv;                       // score width (rk + tail), key-latent rank, value rank
  int alias_v;                          // values are the first rv columns of the key latent
  int num_splits, tiles_per_row, stages;
  float scale_log2;
  const void* qeff;                     // [batch][H][dk], working dtype
  const float* logits;                  // FL mode: fp32 logits [b * lg_sb + h * lg_sh + token] from a first pass
  int64_t lg_sb, lg_sh;
  void* logits_out;                     // logits-only mode: lo_scale * q_eff.k, no softmax / P.V; in the working
  int64_t lo_sb, lo_sh;                 // dtype, or fp32 (lo_f32) when they feed a second pass
  float lo_scale;
  int lo_f32;
  float* partial_o;                     // [batch][H][splits][rv]
  float* lse;                           // [batch][H][splits]
  int* status;
  const int32_t* kv_lens;               // per-row lengths (ragged batches) or NULL
};

__device__ __forceinline__ uint32_t swz(int row, int col_bytes) {
  // byte offset inside a [rows x 128 B] block with the 128-byte TMA swizzle
  return row * 128 + ((((col_bytes >> 4) ^ (row & 7)) << 4) | (col_bytes & 15));
}
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t pack2f(float lo, float hi, __nv_bfloat16) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack2f(float lo, float hi, __half) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack2f(uint32_t u, __nv_bfloat16) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}
__device__ __forceinline__ float2 unpack2f(uint32_t u, __half) {
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}
__device__ __forceinline__ void group_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
// Barrier over the 256 compute threads that also agrees on the abort flag: either all of them
// leave the tile loop or none does.
__device__ __forceinline__ bool group_bar_aborted(volatile int* abort_flag) {
  const uint32_t mine = *abort_flag ? 1u : 0u;
  uint32_t any;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "barrier.cta.red.or.pred q, 1, 256, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(any)
      : "r"(mine)
      : "memory");
  return any != 0;
}

// HB: heads per CTA (32 or 64).  NT: 8-column value n-tiles per warp (rv <= 64 * NT).
// FL: the scores come as fp32 logits from a first pass (reconstructed or dense keys) instead of
//     Q_eff . K^T; only the value latent is streamed.
template <typename T, int HB, int NT, bool FL>
__global__ void __launch_bounds__(NTHREADS, (HB == 32 && NT <= 4) ? 2 : 1)
latent_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmKt,
                 const __grid_constant__ CUtensorMap tmV, const Args a) {
  constexpr int MT = HB / 16;                       // m-tiles of 16 heads
  constexpr int NU = (TILE / 8) * MT;               // (16 heads x 8 tokens) score units per tile
  constexpr int UPW = NU / NCW;                     // units per warp (they share one m-tile)
  static_assert(NU % NCW == 0 && NCW % MT == 0, "unit split");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, hblk = blockIdx.y, b = blockIdx.z;
  const int h0 = hblk * HB;
  const int row_len = a.kv_lens ? min(max(a.kv_lens[b], 0), a.kv_len) : a.kv_len;   // this row's length
  const int row_tiles = a.kv_lens ? (row_len + TILE - 1) / TILE : a.tiles_per_row;
  const int tile_begin = (int)(((int64_t)split * row_tiles) / a.num_splits);
  const int tile_end = (int)(((int64_t)(split + 1) * row_tiles) / a.num_splits);
  const int KB = FL ? 0 : a.dk / 64, KBK = FL ? 0 : a.rk / 64, VB = a.rv / 64;
  const int vblk0 = a.alias_v ? 0 : KB;             // first 64-column block of the value rows in a stage
  const int stage_blocks = a.alias_v ? KB : KB + VB;
  const uint32_t BLK = TILE * 128;                  // bytes of one [32 x 64] block
  const uint32_t stage_bytes = stage_blocks * BLK;

  // shared memory map
  const uint32_t off_q = 0;                                     // HB x dk, blocks of [HB x 128 B]
  const uint32_t q_bytes = (uint32_t)KB * HB * 128;
  const uint32_t off_ring = (q_bytes + 1023u) & ~1023u;
  const uint32_t off_p = off_ring + a.stages * stage_bytes;     // [HB][32 tokens] bf16, 64 B rows
  const uint32_t off_wmax = off_p + HB * 64;                    // [HB][4] floats (per 8-token group)
  const uint32_t off_bar = off_wmax + HB * 16;
  auto bar_full = [&](int s) { return base + off_bar + 8u * s; };
  int* cnt_s = reinterpret_cast<int*>(sm + off_bar + 32);      // per stage: warps that finished reading it
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + off_bar + 64);

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) { mbar_init(bar_full(s), 1); cnt_s[s] = 0; }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  // resident queries: row r, block kb -> swizzled [HB x 128 B] block; rows past num_heads are zero
  if (!FL) {
    const T* qg = static_cast<const T*>(a.qeff) + ((int64_t)b * a.num_heads + h0) * a.dk;
    const int chunks = HB * KB * 8;                 // 16-byte chunks
    for (int c = threadIdx.x; c < chunks; c += NTHREADS) {
      const int r = c / (KB * 8), rem = c - r * (KB * 8), kb = rem >> 3, ch = rem & 7;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (h0 + r < a.num_heads) v = *reinterpret_cast<const uint4*>(qg + (int64_t)r * a.dk + kb * 64 + ch * 8);
      *reinterpret_cast<uint4*>(sm + off_q + kb * (HB * 128) + swz(r, ch * 16)) = v;
    }
  }
  __syncthreads();

  const int g = lane >> 2, t = lane & 3;
  float acc[MT][NT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int n = 0; n < NT; ++n) { acc[m][n][0] = acc[m][n][1] = acc[m][n][2] = acc[m][n][3] = 0.f; }
  float m_run[MT][2];
#pragma unroll
  for (int m = 0; m < MT; ++m) { m_run[m][0] = -CUDART_INF_F; m_run[m][1] = -CUDART_INF_F; }
  float l_run[2] = {0.f, 0.f};
  const int cw = warp;                              // all eight warps compute
  const int mt_w = cw % MT;                         // the m-tile all score units of this warp belong to

  // One thread fills a stage: the tile's key blocks, the tail and (unless aliased) the value blocks.
  auto issue_tile = [&](int tile, int stage) {
    mbar_expect_tx(bar_full(stage), stage_bytes);
    const uint32_t ss = base + off_ring + stage * stage_bytes;
    for (int kb = 0; kb < KBK; ++kb) tma_load_3d(ss + kb * BLK, &tmK, kb * 64, tile * TILE, b, bar_full(stage));
    for (int kb = KBK; kb < KB; ++kb) tma_load_3d(ss + kb * BLK, &tmKt, (kb - KBK) * 64, tile * TILE, b, bar_full(stage));
    if (!a.alias_v)
      for (int vb = 0; vb < VB; ++vb) tma_load_3d(ss + (KB + vb) * BLK, &tmV, vb * 64, tile * TILE, b, bar_full(stage));
  };
  // A warp that is done with a stage fences its reads (generic proxy) against the refill (async
  // proxy) and is counted; the warp that completes the count issues the TMA for the tile that reuses
  // the stage, so no warp is set aside as a producer and nobody waits for a free stage.
  auto release_stage_counted = [&](int tile, int stage) {
    __syncwarp();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (lane == 0) {
      __threadfence_block();
      if (atomicAdd(cnt_s + stage, 1) == NCW - 1) {
        *reinterpret_cast<volatile int*>(cnt_s + stage) = 0;
        __threadfence_block();
        if (tile + a.stages < tile_end) issue_tile(tile + a.stages, stage);
      }
    }
  };
  if (threadIdx.x == 0)
    for (int i = 0; i < a.stages && tile_begin + i < tile_end; ++i) issue_tile(tile_begin + i, i);
  {
    // =========================== compute warps ================================================
    float* wmax_s = reinterpret_cast<float*>(sm + off_wmax);
    int stage = 0;
    uint32_t phase = 0;
    const int mi = lane >> 3, r8 = lane & 7;
    const int nvt = a.rv / 64;                      // value n-tiles this warp really owns (<= NT)
    // FL: logits of this warp's units, fetched one tile ahead (rows g / g+8, tokens 2t / 2t+1)
    float lgn[UPW][4];
    auto fetch_logits = [&](int tile) {
#pragma unroll
      for (int u = 0; u < UPW; ++u) {
        const int j = cw / MT + u * (NCW / MT);
        const int tok = tile * TILE + j * 8 + 2 * t;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int h = h0 + mt_w * 16 + g + (i >> 1) * 8;
          const int tk = tok + (i & 1);
          lgn[u][i] = (tile < tile_end && h < a.num_heads && tk < row_len)
                          ? __ldg(a.logits + (int64_t)b * a.lg_sb + (int64_t)h * a.lg_sh + tk)
                          : 0.f;
        }
      }
    };
    if (FL) fetch_logits(tile_begin);
    for (int tile = tile_begin; tile < tile_end; ++tile) {
      bool ok = mbar_wait(bar_full(stage), phase, abort_flag);
      if (!__all_sync(0xffffffffu, ok) && lane == 0) report(a.status, XKV_ERR_TIMEOUT, 1, tile, hblk, b);
      // (a failed wait raises the abort flag; the warps agree to leave at barrier (A) below)
      const uint32_t ss = base + off_ring + stage * stage_bytes;
      // ---- S units: (m-tile mt_w) x (8-token group j = cw / MT + u * (NCW / MT)) -------------------
      float sc[UPW][4];
#pragma unroll
      for (int u = 0; u < UPW; ++u) { sc[u][0] = sc[u][1] = sc[u][2] = sc[u][3] = 0.f; }
      if (FL) {
#pragma unroll
        for (int u = 0; u < UPW; ++u)
#pragma unroll
          for (int i = 0; i < 4; ++i) sc[u][i] = lgn[u][i];
        fetch_logits(tile + 1);
      }
      for (int kb = 0; kb < KB; ++kb) {
        const uint32_t qb = base + off_q + kb * (HB * 128);
        const uint32_t kblk = ss + kb * BLK;
#pragma unroll
        for (int k2 = 0; k2 < 2; ++k2) {            // two pairs of 16-dim k-steps per 64-column block
          // A fragments (16 heads x 16 dims) for k-steps 2*k2 and 2*k2+1
          uint32_t qa[2][4];
#pragma unroll
          for (int kk = 0; kk < 2; ++kk) {
            const int row = mt_w * 16 + (mi & 1) * 8 + r8;
            const int colb = ((k2 * 2 + kk) * 16 + (mi >> 1) * 8) * 2;
            ldsm4(qb + swz(row, colb), qa[kk]);
          }
#pragma unroll
          for (int u = 0; u < UPW; ++u) {
            const int j = cw / MT + u * (NCW / MT);
            // B fragments: tokens j*8.., dims of the two k-steps: matrices (k lo, k hi) x (step 0, step 1)
            uint32_t kf[4];
            ldsm4(kblk + swz(j * 8 + r8, (k2 * 32 + mi * 8) * 2), kf);
            TypeTraits<T>::mma(sc[u], qa[0], kf[0], kf[1]);
            TypeTraits<T>::mma(sc[u], qa[1], kf[2], kf[3]);
          }
        }
      }
      if (a.logits_out) {
        // logits-only call: store the scaled scores and hand the stage back (no barriers in this mode)
#pragma unroll
        for (int u = 0; u < UPW; ++u) {
          const int j = cw / MT + u * (NCW / MT);
          const int tok = tile * TILE + j * 8 + 2 * t;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int h = h0 + mt_w * 16 + g + (i >> 1) * 8, tk = tok + (i & 1);
            if (h < a.num_heads && tk < row_len) {
              const int64_t off = (int64_t)b * a.lo_sb + (int64_t)h * a.lo_sh + tk;
              if (a.lo_f32) static_cast<float*>(a.logits_out)[off] = sc[u][i] * a.lo_scale;
              else static_cast<T*>(a.logits_out)[off] = TypeTraits<T>::from_f(sc[u][i] * a.lo_scale);
            }
          }
        }
        release_stage_counted(tile, stage);
        if (++stage == a.stages) { stage = 0; phase ^= 1u; }
        if (*abort_flag) break;
        continue;
      }
      // ---- tile max per head -------------------------------------------------------------------------
      float sv[UPW][4];
#pragma unroll
      for (int u = 0; u < UPW; ++u) {
        const int j = cw / MT + u * (NCW / MT);
        const int tok = tile * TILE + j * 8 + 2 * t;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          sv[u][i] = (tok + (i & 1)) < row_len ? sc[u][i] * a.scale_log2 : -CUDART_INF_F;
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          float mx = fmaxf(sv[u][rr * 2], sv[u][rr * 2 + 1]);
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
          if (t == 0) wmax_s[(mt_w * 16 + g + rr * 8) * 4 + j] = mx;
        }
      }
      if (group_bar_aborted(abort_flag)) break;     // (A) unit maxima visible; previous tile's P.V done
      float alpha[MT][2], m_use[MT][2];
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          const float4 w4 = *reinterpret_cast<const float4*>(wmax_s + (m * 16 + g + rr * 8) * 4);
          const float mn = fmaxf(m_run[m][rr], fmaxf(fmaxf(w4.x, w4.y), fmaxf(w4.z, w4.w)));
          m_use[m][rr] = mn == -CUDART_INF_F ? 0.f : mn;
          alpha[m][rr] = exp2f(m_run[m][rr] - m_use[m][rr]);
          m_run[m][rr] = mn;
        }
      // ---- P = exp2(S - m) -> shared memory (rows = heads, 32 tokens = 64 B per row) ----------------
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) l_run[rr] *= alpha[mt_w][rr];
#pragma unroll
      for (int u = 0; u < UPW; ++u) {
        const int j = cw / MT + u * (NCW / MT);
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          const int row = mt_w * 16 + g + rr * 8;
          const uint32_t pk = pack2f(exp2f(sv[u][rr * 2] - m_use[mt_w][rr]), exp2f(sv[u][rr * 2 + 1] - m_use[mt_w][rr]), T());
          const float2 pr = unpack2f(pk, T());
          l_run[rr] += pr.x + pr.y;
          // 64-byte rows: chunk index (0..3) xor-swizzled with the row so ldmatrix reads spread over banks
          const uint32_t off = row * 64 + (((j ^ ((row >> 1) & 3)) << 4) | (t * 4));
          *reinterpret_cast<uint32_t*>(sm + off_p + off) = pk;
        }
      }
      group_bar();                                  // (B) P visible
      // ---- O = O * alpha + P . V : this warp owns value columns [cw * rv/8, (cw+1) * rv/8) -----------
      // the running maxima settle after the first tiles: skip the rescale while no row of the warp moved
      bool moved = false;
#pragma unroll
      for (int m = 0; m < MT; ++m) moved = moved || alpha[m][0] != 1.f || alpha[m][1] != 1.f;
      if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            acc[m][n][0] *= alpha[m][0]; acc[m][n][1] *= alpha[m][0];
            acc[m][n][2] *= alpha[m][1]; acc[m][n][3] *= alpha[m][1];
          }
      }
      if (a.kv_lens != nullptr && (tile + 1) * TILE > row_len) {
        // Ragged batch, last tile of the row: latent rows past the row's own length are outside the
        // call (they may hold anything, NaN included, and 0 * NaN is NaN).  Each warp zeroes its own
        // value columns of those rows; every score read of this tile is behind barrier (B).
        const int first = max(row_len - tile * TILE, 0), chunks = a.rv / 64;
        for (int idx = lane; idx < (TILE - first) * chunks; idx += 32) {
          const int token = first + idx / chunks, col = cw * (a.rv / 8) + (idx % chunks) * 8;
          const uint32_t za = ss + (vblk0 + (col >> 6)) * BLK + swz(token, (col & 63) * 2);
          asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(za), "r"(0u) : "memory");
        }
        __syncwarp();
      }
#pragma unroll
      for (int ks = 0; ks < TILE / 16; ++ks) {
        uint32_t pa[MT][4];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const int row = m * 16 + (mi & 1) * 8 + r8;
          const int chunk = ks * 2 + (mi >> 1);     // 8-token chunk of the row
          ldsm4(base + off_p + row * 64 + ((chunk ^ ((row >> 1) & 3)) << 4), pa[m]);
        }
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
          if (np * 2 < nvt) {
            const int col = cw * (a.rv / 8) + np * 16 + (mi >> 1) * 8;      // value column of this matrix
            const int token = ks * 16 + (mi & 1) * 8 + r8;
            uint32_t vf[4];
            ldsm4t(ss + (vblk0 + (col >> 6)) * BLK + swz(token, (col & 63) * 2), vf);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              TypeTraits<T>::mma(acc[m][np * 2], pa[m], vf[0], vf[1]);
              TypeTraits<T>::mma(acc[m][np * 2 + 1], pa[m], vf[2], vf[3]);
            }
          }
        }
      }
      release_stage_counted(tile, stage);
      if (++stage == a.stages) { stage = 0; phase ^= 1u; }
    }
    // ---- row sums: this thread's partial for rows (mt_w, g) and (mt_w, g + 8) ------------------------
    // Each head row is covered by the NCW / MT warps that share its m-tile; every warp writes its own
    // slot (the per-tile maxima buffer is free now) and the slots are added in a fixed order below,
    // so repeated calls give identical bits.
    float* lpart_s = reinterpret_cast<float*>(sm + off_wmax);      // [HB][NCW / MT]
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      float l = l_run[rr];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      if (t == 0) lpart_s[(mt_w * 16 + g + rr * 8) * (NCW / MT) + cw / MT] = l;
    }
  }
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    return;
  }
  if (a.logits_out == nullptr) {
    const float* lpart_s = reinterpret_cast<const float*>(sm + off_wmax);
    const int H = a.num_heads;
    const int nvt = a.rv / 64;
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const int h = h0 + m * 16 + g + rr * 8;
        if (h < H) {
          float l = 0.f;
#pragma unroll
          for (int k = 0; k < NCW / MT; ++k) l += lpart_s[(m * 16 + g + rr * 8) * (NCW / MT) + k];
          const float inv = l > 0.f ? 1.f / l : 0.f;
          float* po = a.partial_o + (((int64_t)b * H + h) * a.num_splits + split) * a.rv + cw * (a.rv / 8);
#pragma unroll
          for (int n = 0; n < NT; ++n)
            if (n < nvt)
              *reinterpret_cast<float2*>(po + n * 8 + 2 * t) = make_float2(acc[m][n][rr * 2] * inv, acc[m][n][rr * 2 + 1] * inv);
          if (cw == 0 && t == 0)
            a.lse[((int64_t)b * H + h) * a.num_splits + split] =
                l > 0.f ? (m_run[m][rr] + log2f(l)) * 0.6931471805599453f : -CUDART_INF_F;
        }
      }
  }
}

// q_eff[b, h, :] = q . k_proj^T (or a copy of q) followed by the decoupled RoPE query part, in T.
template <typename T>
__global__ void absorb_query_lowp_kernel(const xkv_decode_params p, T* __restrict__ qeff, int dk) {
  extern __shared__ float q_s[];
  const int h = blockIdx.x, b = blockIdx.y;
  const T* q = static_cast<const T*>(p.q) + (int64_t)b * p.q_sb + (int64_t)h * p.q_sh;
  T* out = qeff + ((int64_t)b * p.num_heads + h) * dk;
  for (int d = threadIdx.x; d < p.head_dim; d += blockDim.x) q_s[d] = TypeTraits<T>::to_f(q[d]);
  __syncthreads();
  if (p.k_proj != nullptr) {
    const int div = p.num_heads / p.k_proj_heads;
    const T* kp = static_cast<const T*>(p.k_proj) + (int64_t)b * p.kp_sb + (int64_t)(h / div) * p.kp_sh;
    const bool vec = p.kp_sd == 1 && p.head_dim % 8 == 0 && (reinterpret_cast<uintptr_t>(kp) & 15u) == 0 &&
                     (p.kp_sr * 2) % 16 == 0;
    for (int r = threadIdx.x; r < p.k_rank; r += blockDim.x) {
      const T* rowp = kp + (int64_t)r * p.kp_sr;
      float s = 0.f;
      if (vec) {
        for (int d = 0; d < p.head_dim; d += 8) {
          const uint4 raw = *reinterpret_cast<const uint4*>(rowp + d);
          const T* e8 = reinterpret_cast<const T*>(&raw);
#pragma unroll
          for (int e = 0; e < 8; ++e) s = fmaf(q_s[d + e], TypeTraits<T>::to_f(e8[e]), s);
        }
      } else {
        for (int d = 0; d < p.head_dim; ++d) s = fmaf(q_s[d], TypeTraits<T>::to_f(rowp[(int64_t)d * p.kp_sd]), s);
      }
      out[r] = TypeTraits<T>::from_f(s);
    }
  } else {
    for (int d = threadIdx.x; d < p.k_rank; d += blockDim.x) out[d] = TypeTraits<T>::from_f(q_s[d]);
  }
  if (p.tail_dim > 0) {
    const T* qt = static_cast<const T*>(p.q_tail) + (int64_t)b * p.qt_sb + (int64_t)h * p.qt_sh;
    for (int d = threadIdx.x; d < p.tail_dim; d += blockDim.x) out[p.k_rank + d] = qt[d];
  }
}

bool encode_rows(CUtensorMap* m, int dtype, const void* ptr, int width, int L, int batch, int64_t sl, int64_t sb) {
  const cuuint64_t dims[3] = {(cuuint64_t)width, (cuuint64_t)L, (cuuint64_t)batch};
  const int64_t sbb = batch > 1 ? sb : (int64_t)L * sl;
  const cuuint64_t strides[2] = {(cuuint64_t)sl * 2, (cuuint64_t)sbb * 2};
  const cuuint32_t box[3] = {64, TILE, 1};
  return encode_tiled_16bit(m, dtype, 3, ptr, dims, strides, box);
}

int heads_per_cta(const xkv_decode_params& p) {
  const int dk = p.k_rank + p.tail_dim;
  return (p.num_heads > 32 && p.v_rank <= 512 && dk <= 576) ? 64 : 32;
}

size_t smem_need(const xkv_decode_params& p, int hb, int stages) {
  const int dk = p.k_rank + p.tail_dim;
  const bool alias = p.v == p.k && p.v_sl == p.k_sl && p.v_sb == p.k_sb && p.v_rank <= p.k_rank;
  const size_t q = align_up((size_t)(dk / 64) * hb * 128, 1024);
  const size_t stage = (size_t)((dk / 64) + (alias ? 0 : p.v_rank / 64)) * TILE * 128;
  return q + stages * stage + hb * 64 + hb * 16 + 64 + 16;
}

template <typename T, int HB, int NT, bool FL>
int launch(const CUtensorMap& tK, const CUtensorMap& tKt, const CUtensorMap& tV, const Args& a, int hblocks,
           size_t smem, cudaStream_t st) {
  auto kern = latent_tc_kernel<T, HB, NT, FL>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    cudaGetLastError();
    return XKV_ERR_LAUNCH;
  }
  kern<<<dim3(a.num_splits, hblocks, a.batch), NTHREADS, smem, st>>>(tK, tKt, tV, a);
  return cudaGetLastError() == cudaSuccess ? XKV_OK : XKV_ERR_LAUNCH;
}

template <typename T, bool FL>
int dispatch(int hb, int nt, const CUtensorMap& tK, const CUtensorMap& tKt, const CUtensorMap& tV, const Args& a,
             int hblocks, size_t smem, cudaStream_t st) {
  if (hb == 64) {
    if (nt <= 4) return launch<T, 64, 4, FL>(tK, tKt, tV, a, hblocks, smem, st);
    return launch<T, 64, 8, FL>(tK, tKt, tV, a, hblocks, smem, st);
  }
  if (nt <= 4) return launch<T, 32, 4, FL>(tK, tKt, tV, a, hblocks, smem, st);
  if (nt <= 8) return launch<T, 32, 8, FL>(tK, tKt, tV, a, hblocks, smem, st);
  return launch<T, 32, 16, FL>(tK, tKt, tV, a, hblocks, smem, st);
}

}  // namespace

int launch_absorb_query_lowp(const xkv_decode_params& p, void* qeff, int dk, cudaStream_t st) {
  if (p.dtype == XKV_BF16)
    absorb_query_lowp_kernel<__nv_bfloat16><<<dim3(p.num_heads, p.batch), 128, p.head_dim * sizeof(float), st>>>(
        p, static_cast<__nv_bfloat16*>(qeff), dk);
  else
    absorb_query_lowp_kernel<__half><<<dim3(p.num_heads, p.batch), 128, p.head_dim * sizeof(float), st>>>(
        p, static_cast<__half*>(qeff), dk);
  return cudaGetLastError() == cudaSuccess ? XKV_OK : XKV_ERR_LAUNCH;
}

// A logits-only call is planned as if the values aliased the key latent: nothing but keys is streamed.
static xkv_decode_params normalized(const xkv_decode_params& p) {
  xkv_decode_params t = p;
  if (p.flags & XKV_FLAG_LOGITS_ONLY) {
    t.value_mode = XKV_VALUE_LATENT;
    t.v = p.k; t.v_sl = p.k_sl; t.v_sb = p.k_sb;
    t.v_rank = p.k_rank >= 128 ? 128 : p.k_rank;
    t.v_proj = nullptr;
    t.value_dim = t.v_rank;
  }
  return t;
}

bool latent_tc_supported(const xkv_decode_params& pin) {
  if (pin.score_mode != XKV_SCORE_LATENT) return false;
  const bool lo = (pin.flags & XKV_FLAG_LOGITS_ONLY) != 0;
  if (!lo && pin.value_mode != XKV_VALUE_LATENT) return false;
  if (lo && (pin.k_rank < 128 || (pin.lg_sh < pin.kv_len))) return false;
  const xkv_decode_params p = normalized(pin);
  if (p.dtype != XKV_BF16 && p.dtype != XKV_F16) return false;
  if (p.logit_cap > 0.f) return false;
  if (p.mask) return false;   // additive masks run on the portable kernels
  if (p.k_rank % 64 != 0 || p.v_rank % 128 != 0 || p.tail_dim % 64 != 0) return false;
  if (p.v_rank > 1024 || p.k_rank + p.tail_dim > 1152) return false;
  if (!aligned16(p.k) || !aligned16(p.v) || !stride_ok(p.k_sl) || !stride_ok(p.v_sl)) return false;
  if (p.batch > 1 && (!stride_ok(p.k_sb) || !stride_ok(p.v_sb))) return false;
  if (p.tail_dim > 0 && (!aligned16(p.k_tail) || !stride_ok(p.kt_sl) || (p.batch > 1 && !stride_ok(p.kt_sb)))) return false;
  const int hb = heads_per_cta(p);
  return smem_need(p, hb, 2) <= (size_t)MAX_SMEM;
}

bool latent_tc_plan(const xkv_decode_params& pin, LatentTcPlan* pl) {
  const xkv_decode_params p = normalized(pin);
  const int hb = heads_per_cta(p);
  int stages = 4;
  // the small variant (32 heads, value rank <= 256) is compiled for two CTAs per SM: keep its
  // footprint under half of the shared memory when two stages allow it
  const size_t budget = (hb == 32 && p.v_rank <= 256 && smem_need(p, hb, 2) <= (size_t)MAX_SMEM / 2)
                            ? (size_t)MAX_SMEM / 2 - 1024 : (size_t)MAX_SMEM;
  while (stages > 2 && smem_need(p, hb, stages) > budget) --stages;
  pl->heads_per_cta = hb;
  pl->stages = stages;
  pl->smem_bytes = smem_need(p, hb, stages) + 1024;
  const int tiles = ceil_div(p.kv_len, TILE);
  const int rows = p.batch * ceil_div(p.num_heads, hb);
  const int sms = device_sm_count() * (budget < (size_t)MAX_SMEM ? 2 : 1);   // CTA slots
  int best_s = 1;
  int64_t best_cost = -1;
  const int max_s = tiles < 64 ? tiles : 64;
  for (int s = 1; s <= max_s; ++s) {
    const int64_t waves = ceil_div(rows * s, sms);
    const int64_t cost = waves * (ceil_div(tiles, s) + 4);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_s = s; }
  }
  pl->num_splits = best_s;
  pl->tiles = tiles;
  const int dk = p.k_rank + p.tail_dim;
  size_t off = 256;
  pl->off_qeff = off;
  off += align_up((size_t)p.batch * p.num_heads * dk * 2, 256);
  pl->off_partial = off;
  off += align_up((size_t)p.batch * p.num_heads * best_s * p.v_rank * sizeof(float), 256);
  pl->off_lse = off;
  off += align_up((size_t)p.batch * p.num_heads * best_s * sizeof(float), 256);
  pl->off_olat = 0;
  pl->total_bytes = off;
  return true;
}

int latent_tc_decode(const xkv_decode_params& pin, const LatentTcPlan& pl, void* ws, cudaStream_t st,
                     const LogitsSink* sink) {
  const xkv_decode_params p = normalized(pin);
  const bool lo = (pin.flags & XKV_FLAG_LOGITS_ONLY) != 0;
  char* w = static_cast<char*>(ws);
  const int dk = p.k_rank + p.tail_dim;
  const bool alias = p.v == p.k && p.v_sl == p.k_sl && p.v_sb == p.k_sb && p.v_rank <= p.k_rank;
  CUtensorMap tK, tKt, tV;
  if (!encode_rows(&tK, p.dtype, p.k, p.k_rank, p.kv_len, p.batch, p.k_sl, p.k_sb)) return XKV_ERR_NO_DEVICE;
  if (p.tail_dim > 0) {
    if (!encode_rows(&tKt, p.dtype, p.k_tail, p.tail_dim, p.kv_len, p.batch, p.kt_sl, p.kt_sb)) return XKV_ERR_NO_DEVICE;
  } else {
    tKt = tK;
  }
  if (!alias) {
    if (!encode_rows(&tV, p.dtype, p.v, p.v_rank, p.kv_len, p.batch, p.v_sl, p.v_sb)) return XKV_ERR_NO_DEVICE;
  } else {
    tV = tK;
  }
  int* status = reinterpret_cast<int*>(w);
  clear_status_kernel<<<1, 64, 0, st>>>(status);
  void* qeff = w + pl.off_qeff;
  // a projection shared by the batch is folded into the queries as one tensor-core product over the batch rows
  const int arc = (p.k_proj && p.kp_sb == 0 && batched_projection_fits(p.batch, p.head_dim))
                      ? launch_absorb_query_batched(p, qeff, dk, st)
                      : launch_absorb_query_lowp(p, qeff, dk, st);
  if (arc != XKV_OK) return XKV_ERR_LAUNCH;
  Args a;
  a.batch = p.batch; a.kv_len = p.kv_len; a.num_heads = p.num_heads;
  a.dk = dk; a.rk = p.k_rank; a.rv = p.v_rank; a.alias_v = alias ? 1 : 0;
  a.num_splits = pl.num_splits; a.tiles_per_row = pl.tiles; a.stages = pl.stages;
  a.scale_log2 = p.sm_scale * 1.4426950408889634f;
  a.qeff = qeff;
  a.partial_o = reinterpret_cast<float*>(w + pl.off_partial);
  a.lse = reinterpret_cast<float*>(w + pl.off_lse);
  a.status = status;
  a.kv_lens = p.kv_lens;
  const int hblocks = ceil_div(p.num_heads, pl.heads_per_cta);
  const int nt = p.v_rank / 64;
  a.logits = nullptr; a.lg_sb = a.lg_sh = 0;
  a.logits_out = lo ? pin.logits : nullptr; a.lo_sb = pin.lg_sb; a.lo_sh = pin.lg_sh; a.lo_scale = pin.sm_scale;
  a.lo_f32 = 0;
  if (sink) {   // first pass of a two-pass decode: fp32 logits into the caller's buffer (pin carries XKV_FLAG_LOGITS_ONLY)
    a.logits_out = sink->ptr; a.lo_sb = sink->sb; a.lo_sh = sink->sh; a.lo_f32 = 1;
  }
  const int rc = p.dtype == XKV_BF16
                     ? dispatch<__nv_bfloat16, false>(pl.heads_per_cta, nt, tK, tKt, tV, a, hblocks, pl.smem_bytes, st)
                     : dispatch<__half, false>(pl.heads_per_cta, nt, tK, tKt, tV, a, hblocks, pl.smem_bytes, st);
  if (rc != XKV_OK || lo) return rc;
  // a shared value projection over a few splits: merged while the batch-wide product stages the partial rows
  if (p.v_proj && p.vp_sb == 0 && p.batch >= 4 && !p.lse_out && value_projection_merges(p, pl.num_splits))
    return launch_value_projection_batched(a.partial_o, p, st, a.lse, pl.num_splits);
  return launch_merge(a.partial_o, a.lse, p.out, p.dtype, p.batch, p.num_heads, pl.num_splits, p.v_rank, p.value_dim,
                      p.v_proj, p.v_proj ? p.v_proj_heads : 1, p.vp_sb, p.vp_sh, p.vp_sr, p.vp_sd, p.o_sb, p.o_sh, st, 0, 0,
                      p.lse_out, p.lse_sb);
}

// ---- second pass of the two-pass decode: softmax(logits) . A_v over `heads` stacked heads ----------
// The logits [batch][heads][kv_len] (fp32, already multiplied by sm_scale) come from a first pass
// over reconstructed or dense keys; the value latent (batch, kv_len, v_rank) is streamed once for
// all stacked heads of a head block.  Writes normalised partials + log-sum-exp like the one-pass
// kernel; the caller merges (per layer) and applies the value projections.
bool latent_pv_supported(const xkv_decode_params& p) {
  if (p.value_mode != XKV_VALUE_LATENT || (p.flags & XKV_FLAG_LOGITS_ONLY)) return false;
  if (p.dtype != XKV_BF16 && p.dtype != XKV_F16) return false;
  if (p.v_rank % 128 != 0 || p.v_rank > 1024 || p.logit_cap > 0.f || p.tail_dim != 0) return false;
  if (p.mask) return false;   // additive masks run on the portable kernels
  if (!aligned16(p.v) || !stride_ok(p.v_sl) || (p.batch > 1 && !stride_ok(p.v_sb))) return false;
  return true;
}

bool latent_pv_plan(const xkv_decode_params& p, int heads, LatentTcPlan* pl) {
  const int hb = (heads > 32 && p.v_rank <= 512) ? 64 : 32;
  const size_t stage = (size_t)(p.v_rank / 64) * TILE * 128;
  auto need = [&](int stages) { return stages * stage + hb * 64 + hb * 16 + 64 + 16; };
  int stages = 4;
  while (stages > 2 && need(stages) > (size_t)MAX_SMEM) --stages;
  pl->heads_per_cta = hb;
  pl->stages = stages;
  pl->smem_bytes = need(stages) + 1024;
  const int tiles = ceil_div(p.kv_len, TILE);
  const int rows = p.batch * ceil_div(heads, hb);
  const int sms = device_sm_count();
  int best_s = 1;
  int64_t best_cost = -1;
  const int max_s = tiles < 64 ? tiles : 64;
  for (int s = 1; s <= max_s; ++s) {
    const int64_t waves = ceil_div(rows * s, sms);
    const int64_t cost = waves * (ceil_div(tiles, s) + 4);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_s = s; }
  }
  pl->num_splits = best_s;
  pl->tiles = tiles;
  size_t off = 0;
  pl->off_qeff = off;
  pl->off_partial = off;
  off += align_up((size_t)p.batch * heads * best_s * p.v_rank * sizeof(float), 256);
  pl->off_lse = off;
  off += align_up((size_t)p.batch * heads * best_s * sizeof(float), 256);
  pl->off_olat = 0;
  pl->total_bytes = off;
  return true;
}

int latent_pv_run(const xkv_decode_params& p, int heads, const LatentTcPlan& pl, const float* logits, void* ws,
                  int* status, cudaStream_t st) {
  char* w = static_cast<char*>(ws);
  CUtensorMap tV;
  if (!encode_rows(&tV, p.dtype, p.v, p.v_rank, p.kv_len, p.batch, p.v_sl, p.v_sb)) return XKV_ERR_NO_DEVICE;
  Args a;
  a.batch = p.batch; a.kv_len = p.kv_len; a.num_heads = heads;
  a.dk = 0; a.rk = 0; a.rv = p.v_rank; a.alias_v = 0;
  a.num_splits = pl.num_splits; a.tiles_per_row = pl.tiles; a.stages = pl.stages;
  a.scale_log2 = 1.4426950408889634f;
  a.qeff = nullptr;
  a.logits_out = nullptr; a.lo_sb = a.lo_sh = 0; a.lo_scale = 1.f; a.lo_f32 = 0;
  a.logits = logits; a.lg_sb = (int64_t)heads * p.kv_len; a.lg_sh = p.kv_len;
  a.partial_o = reinterpret_cast<float*>(w + pl.off_partial);
  a.lse = reinterpret_cast<float*>(w + pl.off_lse);
  a.status = status;
  a.kv_lens = p.kv_lens;
  const int hblocks = ceil_div(heads, pl.heads_per_cta);
  const int nt = p.v_rank / 64;
  return p.dtype == XKV_BF16
             ? dispatch<__nv_bfloat16, true>(pl.heads_per_cta, nt, tV, tV, tV, a, hblocks, pl.smem_bytes, st)
             : dispatch<__half, true>(pl.heads_per_cta, nt, tV, tV, tV, a, hblocks, pl.smem_bytes, st);
}

}  // namespace xkv
