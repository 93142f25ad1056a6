// Shared-latent decode (MLA, absorbed factorized caches) on tcgen05, two CTAs per (KV split, head
// block, batch row).
//
// Up to 128 query heads sit on the M dimension of every MMA.  The output rows O[128 x Rv] (fp32)
// alone would fill the 512 tensor-memory columns of an SM, and the resident queries Q[128 x Dk] most
// of its shared memory, so a CLUSTER OF TWO CTAs shares each 32-token tile:
//   * CTA r owns half of the value columns (O[128 x Rv/2] stays in its tensor memory for the whole
//     split) and half of the score contraction: it keeps the matching 64-wide blocks of Q resident,
//     streams only those blocks of the latent rows (each latent byte is fetched by exactly one of the
//     two CTAs, so the pair reads the cache once), and forms S_r = Q_r . K_r^T on the tensor core;
//   * the two partial score tiles are exchanged through distributed shared memory (st.async from registers
//     into the peer's buffer, which counts the bytes on the peer's mbarrier; no multicast, no fences on the
//     sender) and added; both CTAs then
//     hold the same S, run the same softmax (one thread per head row, lazily updated reference
//     maximum as in the two-pass value kernel) and multiply their own value columns: O_r += P . V_r.
// Warps: 0 TMA producer (4-stage ring of whole tiles), 1 MMA issuer (the scores run two tiles ahead of
// P.V: three score buffers in tensor memory, two P buffers in shared memory; its score MMAs are compiled in
// as straight-line code for the usual block counts, since every instruction it spends between two MMAs is
// tensor-core idle time), 2 tensor-memory allocation, 4-11 softmax (two threads per
// head row, 16 tokens of the tile each; a tile's partial scores are sent to the peer one tile early, so
// the exchange hides under the previous tile's exponentials: the softmax chain, not the tensor core or
// HBM, paces this kernel).
// Every wait is bounded; on expiry the CTA raises its abort flag, reports where it gave up, drains,
// frees its tensor memory and leaves (the peer's waits then run out the same way).
#include <algorithm>
#include <type_traits>

#include "sm100_common.cuh"

namespace xkv {
using namespace sm100;
namespace {

constexpr int T = 32;                        // tokens per tile
constexpr int MAXB = 5;                      // 64-column blocks per CTA and tile
constexpr int BLK = T * 128;                 // bytes of one [32 tokens x 64 columns] block
#ifndef XKV_LP_TMEM_P
#define XKV_LP_TMEM_P 1
#endif
// The probabilities P of a tile are the A operand of O += P . V.  Kept in TENSOR memory (written with tcgen05.st by
// the softmax threads, read by the MMA as its tensor-memory operand) they need no shared memory and no proxy fence,
// and the 16 KB they would take there pay for a fifth ring stage.  (0: P through shared memory, four stages.)
constexpr bool kTmemP = XKV_LP_TMEM_P != 0;
constexpr int STAGES = kTmemP ? 5 : 4;
constexpr int QBLK = 128 * 128;              // bytes of one [128 heads x 64 columns] query block
constexpr int NTHREADS = 384;
constexpr int TH = T / 2;                     // tokens per softmax thread (two threads share a head row)
constexpr int OFF_Q = 0;
constexpr int OFF_RING = OFF_Q + MAXB * QBLK;                 // 81920
constexpr int OFF_P = OFF_RING + STAGES * MAXB * BLK;
constexpr int P_BYTES = kTmemP ? 0 : 128 * 128;               // 128 head rows x 128 bytes: two buffers of 32 tokens
constexpr int OFF_X = OFF_P + P_BYTES;                        // partial scores from the peer
constexpr int X_BYTES = (T / 4) * 128 * 16;                   // [T/4][128 rows][4 floats] = 16384
constexpr int XW_BYTES = X_BYTES / 8;                         // one softmax warp's share of an exchange buffer
constexpr int OFF_BAR = OFF_X + 2 * X_BYTES;                  // two exchange buffers, alternating per tile
constexpr int OFF_MISC = OFF_BAR + 24 * 8;
constexpr int OFF_RED = OFF_MISC + 16;                        // [2][128] floats: per-half row maxima / sums
constexpr int SMEM_BYTES = OFF_RED + 1024 + 1024;
static_assert(SMEM_BYTES <= 232448, "shared memory budget exceeded");
static_assert(OFF_RING % 1024 == 0 && BLK % 1024 == 0 && OFF_P % 1024 == 0, "swizzled blocks need 1024-byte alignment");
constexpr float RESCALE_THRESHOLD = 8.f;
constexpr uint32_t S_COL0 = 256;             // tensor-memory columns: O in 0..255, three score buffers of 32 from 256
constexpr int SBUF = 3;
constexpr uint32_t P_COL0 = S_COL0 + SBUF * T;   // two P buffers of T / 2 columns (two 16-bit values per column)
static_assert(P_COL0 + T <= 512, "tensor memory: O, score buffers, P buffers");
#ifndef XKV_LP_SPLIT_ODD
#define XKV_LP_SPLIT_ODD 0
#endif
constexpr bool kSplitOddBlock = XKV_LP_SPLIT_ODD != 0;   // an odd score block out is loaded by both CTAs, each scoring half of it

// The 64-column blocks one CTA of the pair works on.  Blocks [0, nv) are its own value columns (in
// alias mode they are score blocks too); blocks with score[i] set take part in S.
struct BlockList {
  int n, nv;
  int col[MAXB];        // column (elements) inside the tensor the block is loaded from
  int src[MAXB];        // 0: key latent, 1: decoupled RoPE key part, 2: value latent
  int qcol[MAXB];       // matching column of the effective query, or -1 when the block is values only
  int ks0;              // first score block of the list (value-only blocks come before it)
  uint32_t steps;       // which 16-column MMA steps of the score blocks this CTA issues: bit 4 * (i - ks0) + k4
};

struct Args {
  int batch, kv_len, num_heads, dk;
  int num_splits, tiles_per_row;
  float scale_log2;
  const void* qeff;                       // [batch][H][dk], working dtype; null: the two parts are read where the caller has them
  const void* q;                          // columns [0, q_cols) of a query row: q + b * q_sb + h * q_sh
  const void* q_tail;                     // columns [q_cols, dk): q_tail + b * qt_sb + h * qt_sh
  int64_t q_sb, q_sh, qt_sb, qt_sh;
  int q_cols;
  void* out;                              // not null (one split only): finished rows in the working dtype, out + b * o_sb + h * o_sh
  int64_t o_sb, o_sh;
  float* partial_o;                       // [batch][H][splits][rv]
  float* lse;                             // [batch][H][splits]
  int rv;
  int* status;
  const int32_t* kv_lens;
  BlockList bl[2];
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Bounded wait whose acquire covers writes made by the other CTA of the cluster.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  const uint64_t t0 = global_ns();
  for (uint32_t it = 0; it < MAX_POLLS; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((it & 31u) == 31u) {
      if (*abort_flag) return false;
      if (global_ns() - t0 > WAIT_LIMIT_NS) break;
      __nanosleep(32);
    }
  }
  *abort_flag = 1;
  return false;
}

#ifdef XKV_TC_PROFILE
// Debug build only: cycles spent in each kind of wait, summed over CTAs into status[8 + 2 * slot] (64-bit).
#define XKV_LP_WAIT(slot, leader, expr)                                              \
  [&]() {                                                                            \
    const long long t0_ = clock64();                                                 \
    const bool r_ = (expr);                                                          \
    if (leader)                                                                      \
      atomicAdd(reinterpret_cast<unsigned long long*>(a.status + 8) + (slot),        \
                (unsigned long long)(clock64() - t0_));                              \
    return r_;                                                                       \
  }()
#define XKV_LP_MARK(slot)                                                                         \
  do {                                                                                            \
    const long long now_ = clock64();                                                             \
    if (threadIdx.x == 128) atomicAdd(reinterpret_cast<unsigned long long*>(a.status + 8) + (slot), (unsigned long long)(now_ - mark_)); \
    mark_ = now_;                                                                                 \
  } while (0)
#else
#define XKV_LP_WAIT(slot, leader, expr) (expr)
#define XKV_LP_MARK(slot) do { } while (0)
#endif

template <typename T_>
__global__ void __launch_bounds__(NTHREADS, 1)
latent_pair_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmKt,
                   const __grid_constant__ CUtensorMap tmV, const Args a) {
  extern __shared__ uint8_t smem_raw[];
#ifdef XKV_TC_PROFILE
  const long long t_entry_ = clock64();
#endif
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank(), peer = rank ^ 1u;
  const int hb = blockIdx.x >> 1, b = blockIdx.y, split = blockIdx.z;
  const BlockList& bl = a.bl[rank];
  const int h0 = hb * 128;
  const int row_len = a.kv_lens ? min(max(a.kv_lens[b], 0), a.kv_len) : a.kv_len;
  const int row_tiles = a.kv_lens ? (row_len + T - 1) / T : a.tiles_per_row;
  const int tile_begin = (int)(((int64_t)split * row_tiles) / a.num_splits);
  const int tile_end = (int)(((int64_t)(split + 1) * row_tiles) / a.num_splits);
  const int ntiles = tile_end - tile_begin;
  const int nvc = bl.nv * 64;                               // value columns of this CTA
  const int col_out = (int)rank * (a.rv / 2);               // where they sit in the output row
  const uint32_t stage_bytes = (uint32_t)bl.n * BLK;

  const uint32_t bar0 = base + OFF_BAR;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };                       // [STAGES] a tile's blocks have landed
  auto bar_empty = [&](int s) { return bar0 + 8u * (STAGES + s); };           // [STAGES] P.V of the tile that used the stage has run
  auto bar_sfull = [&](int i) { return bar0 + 8u * (2 * STAGES + i); };       // [SBUF] a score buffer holds S of a tile
  auto bar_sempty = [&](int i) { return bar0 + 8u * (2 * STAGES + SBUF + i); };   // [SBUF] the softmax threads have read it
  constexpr int kBarP = 2 * STAGES + 2 * SBUF;
  auto bar_pfull = [&](int i) { return bar0 + 8u * (kBarP + i); };            // [2] a P buffer holds the probabilities of a tile
  auto bar_pempty = [&](int i) { return bar0 + 8u * (kBarP + 2 + i); };       // [2] P.V of the tile that used it has run
  const uint32_t bar_odone = bar0 + 8u * (kBarP + 4);
  auto bar_xfull = [&](int i) { return bar0 + 8u * (kBarP + 5 + i); };        // [2] the peer's partial scores have landed in exchange buffer i
  static_assert(kBarP + 7 <= 24, "barrier slots");
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_MISC + 4);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
    for (int i = 0; i < SBUF; ++i) { mbar_init(bar_sfull(i), 1); mbar_init(bar_sempty(i), 256); }
    for (int i = 0; i < 2; ++i) { mbar_init(bar_pfull(i), 256); mbar_init(bar_pempty(i), 1); }
    mbar_init(bar_odone, 1);
    for (int i = 0; i < 2; ++i) mbar_init(bar_xfull(i), 1);   // one local arrive.expect_tx per use + the peer's st.async bytes
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(base + OFF_MISC), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // resident queries: the score blocks of this CTA, rows past num_heads are zero
  {
    const T_* qg = static_cast<const T_*>(a.qeff) + ((int64_t)b * a.num_heads + h0) * a.dk;
    // the score blocks are the last ones of the list, query block qi belongs to list entry ks0 + qi; four
    // 16-byte loads are in flight per thread before the first one is stored
    const int nq = (bl.n - bl.ks0) * 1024;
    for (int i0 = threadIdx.x; i0 < nq; i0 += 4 * NTHREADS) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = i0 + u * NTHREADS;
        v[u] = make_uint4(0, 0, 0, 0);
        if (idx < nq) {
          const int qi = idx >> 10, r = (idx >> 3) & 127, ch = idx & 7;
          if (h0 + r < a.num_heads) {
            const int col = bl.qcol[bl.ks0 + qi] + ch * 8;
            if (a.qeff != nullptr)
              v[u] = *reinterpret_cast<const uint4*>(qg + (int64_t)r * a.dk + col);
            else if (col < a.q_cols)
              v[u] = *reinterpret_cast<const uint4*>(static_cast<const T_*>(a.q) + (int64_t)b * a.q_sb + (int64_t)(h0 + r) * a.q_sh + col);
            else
              v[u] = *reinterpret_cast<const uint4*>(static_cast<const T_*>(a.q_tail) + (int64_t)b * a.qt_sb + (int64_t)(h0 + r) * a.qt_sh + (col - a.q_cols));
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = i0 + u * NTHREADS;
        if (idx < nq) {
          const int qi = idx >> 10, r = (idx >> 3) & 127, ch = idx & 7;
          *reinterpret_cast<uint4*>(sm + OFF_Q + qi * QBLK + r * 128 + ((ch ^ (r & 7)) << 4)) = v[u];
        }
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> tensor-core reads
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // the peer's barriers exist before anything is signalled across CTAs
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
#ifdef XKV_TC_PROFILE
  const long long t_start_ = clock64();
  const uint64_t ns_start_ = global_ns();
  long long t_loop_end_ = t_start_, t_odone_ = t_start_;
  if (threadIdx.x == 128) atomicAdd(reinterpret_cast<unsigned long long*>(a.status + 8) + 18, (unsigned long long)(t_start_ - t_entry_));
#endif

  if (warp == 0) {
    // =========================== producer: whole tiles of this CTA's blocks ========================
    if (lane == 0) {
      for (int i = 0; i < ntiles; ++i) {
        const int stage = i % STAGES;
        if (!XKV_LP_WAIT(0, true, mbar_wait(bar_empty(stage), ((uint32_t)(i / STAGES) & 1u) ^ 1u, abort_flag))) {
          report(a.status, XKV_ERR_TIMEOUT, 30, tile_begin + i, (int)rank, b);
          break;
        }
        mbar_expect_tx(bar_full(stage), stage_bytes);
        const uint32_t ss = base + OFF_RING + stage * (MAXB * BLK);
        const int tok = (tile_begin + i) * T;
        for (int k = 0; k < bl.n; ++k) {
          const CUtensorMap* m = bl.src[k] == 0 ? &tmK : (bl.src[k] == 1 ? &tmKt : &tmV);
          tma_load_3d(ss + k * BLK, m, bl.col[k], tok, b, bar_full(stage));
        }
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================================================
    if (lane == 0 && ntiles > 0) {
      const uint32_t kfmt = TypeTraits<T_>::kFmt;
      // S = Q . K^T: both operands K-major, N = 48 tokens; O += P . V: A = P K-major, B = values MN-major
      const uint32_t idesc_s = (1u << 4) | (kfmt << 7) | (kfmt << 10) | (((uint32_t)T >> 3) << 17) | ((128u >> 4) << 24);
      const uint32_t idesc_o = (1u << 4) | (kfmt << 7) | (kfmt << 10) | (1u << 16) | (((uint32_t)nvc >> 3) << 17) |
                               ((128u >> 4) << 24);
      // operand descriptors built once; the loops only add offsets
      const uint64_t dq0 = smem_desc(base + OFF_Q, 16, 1024), dk0 = smem_desc(base + OFF_RING, 16, 1024);
      const uint64_t dp0 = smem_desc(base + OFF_P, 16, 1024), dv0 = smem_desc(base + OFF_RING, BLK, 1024);
      (void)dp0;
      // One thread issues every MMA, and what it spends per instruction on addresses and loop control is time the
      // tensor core idles (a 128 x 32 x 16 MMA takes 46 cycles): the usual step sets are compiled in, fully
      // unrolled with constant offsets; any other set runs the loop at the end.
      const uint64_t dks = desc_advance(dk0, (uint32_t)(bl.ks0 * BLK));
      auto issue_scores = [&](auto steps_c, int i) -> bool {
        constexpr uint32_t STEPS = decltype(steps_c)::value;
        const int stage = i % STAGES, sb = i % SBUF;
        if (i >= SBUF && !XKV_LP_WAIT(1, true, mbar_wait(bar_sempty(sb), ((uint32_t)(i / SBUF) & 1u) ^ 1u, abort_flag))) return false;
        if (!XKV_LP_WAIT(2, true, mbar_wait(bar_full(stage), (uint32_t)(i / STAGES) & 1u, abort_flag))) return false;
        tc_fence_after();
        const uint32_t tacc = tmem_base + S_COL0 + (uint32_t)sb * (uint32_t)T;
        const uint64_t db_st = desc_advance(dks, (uint32_t)(stage * (MAXB * BLK)));
        if constexpr (STEPS != 0u) {
#pragma unroll
          for (int j = 0; j < 4 * MAXB; ++j)
            if ((STEPS >> j) & 1u)
              tc_mma(tacc, desc_advance(dq0, (uint32_t)((j >> 2) * QBLK + (j & 3) * 32)),
                     desc_advance(db_st, (uint32_t)((j >> 2) * BLK + (j & 3) * 32)), idesc_s, (STEPS & ((1u << j) - 1u)) ? 1u : 0u);
        } else {
          uint32_t acc = 0u;
          for (int j = 0; j < 4 * MAXB; ++j)
            if ((bl.steps >> j) & 1u) {
              tc_mma(tacc, desc_advance(dq0, (uint32_t)((j >> 2) * QBLK + (j & 3) * 32)),
                     desc_advance(db_st, (uint32_t)((j >> 2) * BLK + (j & 3) * 32)), idesc_s, acc);
              acc = 1u;
            }
        }
        tc_commit(bar_sfull(sb));
        return true;
      };
      // the scores run two tiles ahead of P.V: S(i+2) is in the queue before P of tile i is waited for, so the
      // softmax threads find S(i+1) finished when they turn to it in the middle of tile i
      auto run = [&](auto steps_c) -> bool {
        bool ok = issue_scores(steps_c, 0);
        if (ok && ntiles > 1) ok = issue_scores(steps_c, 1);
        for (int i = 0; ok && i < ntiles; ++i) {
          if (i + 2 < ntiles) ok = issue_scores(steps_c, i + 2);
          if (!ok) break;
          if (!XKV_LP_WAIT(3, true, mbar_wait(bar_pfull(i & 1), (uint32_t)(i >> 1) & 1u, abort_flag))) { ok = false; break; }
          tc_fence_after();
          const uint64_t dv_st = desc_advance(dv0, (uint32_t)((i % STAGES) * (MAXB * BLK)));
          if constexpr (kTmemP) {
            const uint32_t tp = tmem_base + P_COL0 + (uint32_t)((i & 1) * (T / 2));
#pragma unroll
            for (int k4 = 0; k4 < T / 16; ++k4)
              tc_mma_ts(tmem_base, tp + (uint32_t)(k4 * 8), desc_advance(dv_st, k4 * 2048), idesc_o, (i == 0 && k4 == 0) ? 0u : 1u);
          } else {
            const uint64_t dp_i = desc_advance(dp0, (uint32_t)((i & 1) * 64));     // the two P buffers are the halves of the 128-byte rows
#pragma unroll
            for (int k4 = 0; k4 < T / 16; ++k4)
              tc_mma(tmem_base, desc_advance(dp_i, k4 * 32), desc_advance(dv_st, k4 * 2048), idesc_o, (i == 0 && k4 == 0) ? 0u : 1u);
          }
          tc_commit(bar_empty(i % STAGES));      // the tile's blocks and ...
          tc_commit(bar_pempty(i & 1));          // ... its P buffer are free once these MMAs have run
        }
        return ok;
      };
      bool ok;
      switch (bl.steps) {
        case 0xFFFFu: ok = run(std::integral_constant<uint32_t, 0xFFFFu>{}); break;       // four whole blocks
        case 0xFFFFFu: ok = run(std::integral_constant<uint32_t, 0xFFFFFu>{}); break;     // five whole blocks
        case 0x3FFFFu: ok = run(std::integral_constant<uint32_t, 0x3FFFFu>{}); break;     // four blocks and the first half of a fifth
        case 0xCFFFFu: ok = run(std::integral_constant<uint32_t, 0xCFFFFu>{}); break;     // four blocks and the second half of a fifth
        default: ok = run(std::integral_constant<uint32_t, 0u>{}); break;
      }
      if (ok) tc_commit(bar_odone);
      else report(a.status, XKV_ERR_TIMEOUT, 31, tile_begin, (int)rank, b);
    }
  } else if (warp >= 4) {
    // =========================== softmax: two threads per head row, 16 tokens of the tile each =========
    const int r = (threadIdx.x - 128) & 127;                 // head row = tensor-memory lane
    const int half = (threadIdx.x - 128) >> 7;               // warps 4-7: tokens 0-15, warps 8-11: tokens 16-31
    const int h = h0 + r;
    const bool live = h < a.num_heads;
    const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    // exchange buffers: [buffer 2][softmax warp 8][group of 4 tokens][lane][4 floats]: a warp's share is 2 KB in one piece
    const uint32_t x_warp = base + OFF_X + (uint32_t)(warp - 4) * XW_BYTES;          // + buffer * X_BYTES
    const uint32_t x_local = x_warp + (uint32_t)lane * 16u;                             // + g * 512
    const uint32_t x_local_peer = map_to_cta(x_local, peer);
    float* red_s = reinterpret_cast<float*>(sm + OFF_RED);   // [2][128]: per-half row maxima / row sums
    float m_ref = -CUDART_INF_F, l_sum = 0.f;                // l_sum: this thread's tokens only
    bool alive = true;
    // My partial scores of a tile leave tensor memory and go to the peer one tile EARLY (in the middle of
    // the previous tile's softmax), so the exchange's latency hides under that tile's exponentials.  Two
    // exchange buffers with a barrier each.  The partial of tile t goes straight from registers into the
    // PEER's buffer t & 1 (st.async: 16 bytes per store, counted on the peer's barrier; no staging copy and
    // no proxy fence on the sender).  That buffer is free: the peer's partial of tile t - 1 has reached me,
    // and every peer thread sends it only after reading tile t - 2 out of the same buffer.
    float s[TH], s_next[TH];
    auto fetch_and_send = [&](int i) {
      const int sb = i % SBUF;
      if (!XKV_LP_WAIT(4, threadIdx.x == 128, mbar_wait(bar_sfull(sb), (uint32_t)(i / SBUF) & 1u, abort_flag))) report(a.status, XKV_ERR_TIMEOUT, 32, tile_begin + i, (int)rank, b);
      tc_fence_after();
      uint32_t v0[16];
      static_assert(TH == 16, "one 16-column load per thread and tile");
      tmem_ld16(lane_addr + S_COL0 + (uint32_t)sb * (uint32_t)T + (uint32_t)(half * TH), v0);
      tmem_wait_ld();
#pragma unroll
      for (int e = 0; e < 16; ++e) s_next[e] = __uint_as_float(v0[e]);
      tc_fence_before();
      mbar_arrive(bar_sempty(sb));
      const uint32_t dst_off = (uint32_t)(i & 1) * X_BYTES;
      if (threadIdx.x == 128) mbar_expect_tx(bar_xfull(i & 1), X_BYTES);   // my buffer i & 1: all of the peer's bytes for tile i
      {
        const uint32_t bar_peer = map_to_cta(bar_xfull(i & 1), peer);
#pragma unroll
        for (int g4 = 0; g4 < TH / 4; ++g4)
          asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
                       ::"r"(x_local_peer + dst_off + g4 * 512), "r"(__float_as_uint(s_next[4 * g4])), "r"(__float_as_uint(s_next[4 * g4 + 1])),
                         "r"(__float_as_uint(s_next[4 * g4 + 2])), "r"(__float_as_uint(s_next[4 * g4 + 3])), "r"(bar_peer) : "memory");
      }
    };
    if (ntiles > 0) fetch_and_send(0);
    for (int i = 0; i < ntiles && alive; ++i) {
#ifdef XKV_TC_PROFILE
      long long mark_ = clock64();
#endif
#pragma unroll
      for (int e = 0; e < TH; ++e) s[e] = s_next[e];
      // ---- the peer's partial of this tile (sent a tile ago) + mine ------------------------------------
      const uint32_t xoff = (uint32_t)(i & 1) * X_BYTES;
      if (!XKV_LP_WAIT(6, threadIdx.x == 128, mbar_wait_cluster(bar_xfull(i & 1), (uint32_t)(i >> 1) & 1u, abort_flag))) report(a.status, XKV_ERR_TIMEOUT, 34, tile_begin + i, (int)rank, b);
      const int t0 = (tile_begin + i) * T + half * TH;       // first token of this thread
      XKV_LP_MARK(12);
#pragma unroll
      for (int g4 = 0; g4 < TH / 4; ++g4) {
        float4 o;
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(o.x), "=f"(o.y), "=f"(o.z), "=f"(o.w) : "r"(x_local + xoff + g4 * 512));
        // (a + b == b + a exactly: both CTAs end up with the same bits)
        s[4 * g4] = (s[4 * g4] + o.x) * a.scale_log2;
        s[4 * g4 + 1] = (s[4 * g4 + 1] + o.y) * a.scale_log2;
        s[4 * g4 + 2] = (s[4 * g4 + 2] + o.z) * a.scale_log2;
        s[4 * g4 + 3] = (s[4 * g4 + 3] + o.w) * a.scale_log2;
      }
      XKV_LP_MARK(13);
      // ---- next tile's partial on its way while this tile's softmax runs --------------------------------
      if (i + 1 < ntiles) fetch_and_send(i + 1);
      XKV_LP_MARK(11);
      if (t0 + TH > row_len || !live) {
#pragma unroll
        for (int e = 0; e < TH; ++e)
          if (t0 + e >= row_len || !live) s[e] = -CUDART_INF_F;
      }
      float tmax = -CUDART_INF_F;
#pragma unroll
      for (int e = 0; e < TH; ++e) tmax = fmaxf(tmax, s[e]);
      XKV_LP_MARK(10);
      // ---- lazily updated reference maximum: does ANY thread see a score that tops its row's reference by
      // more than the threshold (or a first finite score)?  All 256 agree through one reducing barrier.
      const bool move_hint = tmax > m_ref + RESCALE_THRESHOLD || (m_ref == -CUDART_INF_F && tmax > -CUDART_INF_F);
      // (one barrier per tile: a raised abort flag rides on the same vote and is told apart by a second, rare one)
      auto vote = [](uint32_t mine) -> uint32_t {
        uint32_t r;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.u32 p, %1, 0;\n\t"
            "barrier.cta.red.or.pred q, 1, 256, p;\n\t"
            "selp.u32 %0, 1, 0, q;\n\t}"
            : "=r"(r)
            : "r"(mine)
            : "memory");
        return r;
      };
      const uint32_t anym = vote((move_hint || *abort_flag) ? 1u : 0u);
      if (anym && vote(*abort_flag ? 1u : 0u)) { alive = false; break; }
      XKV_LP_MARK(14);
      // this tile's P buffer is free once P.V of the tile before last has run; a rescale of the output rows has to
      // wait for the previous tile's P.V as well
      if (i > 1 && !XKV_LP_WAIT(7, threadIdx.x == 128, mbar_wait(bar_pempty(i & 1), (uint32_t)((i >> 1) - 1) & 1u, abort_flag))) report(a.status, XKV_ERR_TIMEOUT, 35, tile_begin + i, (int)rank, b);
      if (anym) {
        if (i > 0 && !mbar_wait(bar_pempty((i - 1) & 1), (uint32_t)((i - 1) >> 1) & 1u, abort_flag)) report(a.status, XKV_ERR_TIMEOUT, 38, tile_begin + i, (int)rank, b);
        // rare: the two threads of a row put their maxima together, every row decides for itself, and each
        // thread rescales its half of the row's output columns in tensor memory
        red_s[half * 128 + r] = tmax;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        const float rmax = fmaxf(red_s[r], red_s[128 + r]);
        asm volatile("bar.sync 1, 256;" ::: "memory");        // (the slots are reused by the next rescale)
        const bool move = rmax > m_ref + RESCALE_THRESHOLD || (m_ref == -CUDART_INF_F && rmax > -CUDART_INF_F);
        const float m_new = move ? rmax : m_ref;
        const float alpha = (m_ref == -CUDART_INF_F) ? 0.f : ex2_approx(m_ref - m_new);
        if (i > 0) {
          tc_fence_after();
          const int c0 = half * (nvc / 2);
          for (int c = c0; c < c0 + nvc / 2; c += 32) {
            uint32_t v[32];
            tmem_ld32(lane_addr + c, v);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
            tmem_st32(lane_addr + c, v);
          }
          tmem_wait_st();
          tc_fence_before();
        }
        l_sum *= alpha;
        m_ref = m_new;
      }
      XKV_LP_MARK(15);
      // ---- P row -> tensor memory (or shared memory, K-major with 128-byte swizzle), row sum of the rounded values
      const float mref = m_ref == -CUDART_INF_F ? 0.f : m_ref;
      if constexpr (kTmemP) {
        tc_fence_after();     // the P buffer was released through an mbarrier (tcgen05.commit of the MMAs that read it)
        // lane = head row; a 32-bit column holds two consecutive tokens, this thread's 16 tokens are 8 columns
        uint32_t pk[TH / 2];
#pragma unroll
        for (int e = 0; e < TH / 2; ++e) {
          pk[e] = TypeTraits<T_>::pack2(ex2_approx(s[2 * e] - mref), ex2_approx(s[2 * e + 1] - mref));
          const float2 q = TypeTraits<T_>::unpack2(pk[e]);
          l_sum += q.x + q.y;
        }
        static_assert(TH == 16, "eight packed columns per thread");
        tmem_st8(lane_addr + P_COL0 + (uint32_t)((i & 1) * (T / 2) + half * (TH / 2)), pk);
      } else {
        uint8_t* prow = sm + OFF_P + r * 128;
#pragma unroll
        for (int c8 = 0; c8 < TH / 8; ++c8) {
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            pk[e] = TypeTraits<T_>::pack2(ex2_approx(s[c8 * 8 + 2 * e] - mref), ex2_approx(s[c8 * 8 + 2 * e + 1] - mref));
            const float2 q = TypeTraits<T_>::unpack2(pk[e]);
            l_sum += q.x + q.y;
          }
          *reinterpret_cast<uint4*>(prow + ((((i & 1) * 4 + half * (TH / 8) + c8) ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
      }
      // ragged batch, last tile of the row: value rows past the row's own length may hold anything (NaN
      // included, and 0 * NaN is NaN): zero them before the MMAs read the tile
      const int tile0 = (tile_begin + i) * T;
      if (a.kv_lens != nullptr && tile0 + T > row_len) {
        const int stage = i % STAGES;
        if (!mbar_wait(bar_full(stage), (uint32_t)(i / STAGES) & 1u, abort_flag)) report(a.status, XKV_ERR_TIMEOUT, 36, tile_begin + i, (int)rank, b);
        const int first = max(row_len - tile0, 0), per_row = bl.nv * 8;
        for (int idx = threadIdx.x - 128; idx < (T - first) * per_row; idx += 256) {
          const int row = first + idx / per_row, rem = idx % per_row;
          *reinterpret_cast<uint4*>(sm + OFF_RING + stage * (MAXB * BLK) + (rem >> 3) * BLK + row * 128 + (rem & 7) * 16) =
              make_uint4(0u, 0u, 0u, 0u);
        }
      }
      XKV_LP_MARK(16);
      if constexpr (kTmemP) {
        // only the zeroed tail rows above are generic writes that the tensor core reads through the async proxy
        if (a.kv_lens != nullptr && tile0 + T > row_len) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        tmem_wait_st();
        tc_fence_before();
      } else {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> tensor-core reads
      }
      mbar_arrive(bar_pfull(i & 1));
      XKV_LP_MARK(17);
    }
    // ---- output: O row / l, log-sum-exp; each thread writes its half of the row's columns ---------------
#ifdef XKV_TC_PROFILE
    t_loop_end_ = clock64();
#endif
    if (alive && ntiles > 0) {
      if (!mbar_wait(bar_odone, 0, abort_flag)) report(a.status, XKV_ERR_TIMEOUT, 37, tile_end, (int)rank, b);
      tc_fence_after();
    }
#ifdef XKV_TC_PROFILE
    t_odone_ = clock64();
#endif
    red_s[half * 128 + r] = l_sum;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (alive && !*abort_flag) {
      const float l_row = red_s[r] + red_s[128 + r];          // fixed order: identical in both threads and both CTAs
      const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
      const int c0 = half * (nvc / 2);
      float* po = a.partial_o + (((int64_t)b * a.num_heads + (live ? h : 0)) * a.num_splits + split) * a.rv + col_out;
      for (int c = c0; c < c0 + nvc / 2; c += 32) {
        uint32_t v[32];
        if (ntiles > 0) {                    // (warp-wide tensor-memory load: rows past the last head take part)
          tmem_ld32(lane_addr + c, v);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = 0u;
        }
        if (live && a.out != nullptr) {
          // the only split of its row: the normalised row is the result, stored in the working dtype
          T_* orow = static_cast<T_*>(a.out) + (int64_t)b * a.o_sb + (int64_t)h * a.o_sh + col_out + c;
#pragma unroll
          for (int e = 0; e < 32; e += 8)
            *reinterpret_cast<uint4*>(orow + e) =
                make_uint4(TypeTraits<T_>::pack2(__uint_as_float(v[e]) * inv, __uint_as_float(v[e + 1]) * inv),
                           TypeTraits<T_>::pack2(__uint_as_float(v[e + 2]) * inv, __uint_as_float(v[e + 3]) * inv),
                           TypeTraits<T_>::pack2(__uint_as_float(v[e + 4]) * inv, __uint_as_float(v[e + 5]) * inv),
                           TypeTraits<T_>::pack2(__uint_as_float(v[e + 6]) * inv, __uint_as_float(v[e + 7]) * inv));
        } else if (live) {
#pragma unroll
          for (int e = 0; e < 32; e += 4)
            *reinterpret_cast<float4*>(po + c + e) =
                make_float4(__uint_as_float(v[e]) * inv, __uint_as_float(v[e + 1]) * inv,
                            __uint_as_float(v[e + 2]) * inv, __uint_as_float(v[e + 3]) * inv);
        }
      }
      if (live && rank == 0 && half == 0)
        a.lse[((int64_t)b * a.num_heads + h) * a.num_splits + split] =
            l_row > 0.f ? (m_ref + log2f(l_row)) * 0.6931471805599453f : -CUDART_INF_F;
    }
  }

#ifdef XKV_TC_PROFILE
  if (threadIdx.x == 128)
    atomicAdd(reinterpret_cast<unsigned long long*>(a.status + 8) + 8, (unsigned long long)(clock64() - t_start_));
  if (threadIdx.x == 128) {
    atomicAdd(reinterpret_cast<unsigned long long*>(a.status + 8) + 9, (unsigned long long)(global_ns() - ns_start_));
    atomicAdd(reinterpret_cast<unsigned long long*>(a.status + 8) + 19, (unsigned long long)(t_loop_end_ - t_start_));
    atomicAdd(reinterpret_cast<unsigned long long*>(a.status + 8) + 20, (unsigned long long)(t_odone_ - t_loop_end_));
    atomicAdd(reinterpret_cast<unsigned long long*>(a.status + 8) + 21, (unsigned long long)(clock64() - t_odone_));
  }
#endif
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  // neither CTA leaves while the other may still store into its shared memory or signal its barriers
  cluster_sync_all();
  if (warp == 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

bool encode_rows(CUtensorMap* m, int dtype, const void* ptr, int width, int L, int batch, int64_t sl, int64_t sb) {
  const cuuint64_t dims[3] = {(cuuint64_t)width, (cuuint64_t)L, (cuuint64_t)batch};
  const int64_t sbb = batch > 1 ? sb : (int64_t)L * sl;
  const cuuint64_t strides[2] = {(cuuint64_t)sl * 2, (cuuint64_t)sbb * 2};
  const cuuint32_t box[3] = {64, T, 1};
  return encode_tiled_16bit(m, dtype, 3, ptr, dims, strides, box);
}

bool aliased(const xkv_decode_params& p) {
  return p.v == p.k && p.v_sl == p.k_sl && p.v_sb == p.k_sb && p.v_rank <= p.k_rank;
}

// Split the 64-column blocks of a call between the two CTAs: each takes half of the value columns
// (and, in alias mode, scores those same blocks); the remaining score blocks are dealt out so that
// the two lists are as even as possible.  Returns false when a CTA would need more than MAXB blocks.
bool make_lists(const xkv_decode_params& p, BlockList out[2]) {
  const bool al = aliased(p);
  const int nvb = p.v_rank / 64, kb = p.k_rank / 64, tb = p.tail_dim / 64;
  for (int r = 0; r < 2; ++r) {
    BlockList& l = out[r];
    l.n = 0;
    l.nv = nvb / 2;
    for (int i = 0; i < l.nv; ++i) {
      const int blk = r * l.nv + i;
      l.col[l.n] = blk * 64;
      l.src[l.n] = al ? 0 : 2;
      l.qcol[l.n] = al ? blk * 64 : -1;
      ++l.n;
    }
  }
  // score blocks not covered above: all key blocks (separate value latent) or the key blocks past the
  // value columns (alias), then the decoupled RoPE blocks
  int k4_lo[2][MAXB], k4_hi[2][MAXB];
  for (int r = 0; r < 2; ++r)
    for (int i = 0; i < MAXB; ++i) { k4_lo[r][i] = 0; k4_hi[r][i] = 4; }
  auto put = [&](int r, int blk, int lo, int hi) {
    BlockList& l = out[r];
    if (l.n >= MAXB) return false;
    if (blk < kb) { l.col[l.n] = blk * 64; l.src[l.n] = 0; }
    else { l.col[l.n] = (blk - kb) * 64; l.src[l.n] = 1; }
    l.qcol[l.n] = blk * 64;
    k4_lo[r][l.n] = lo; k4_hi[r][l.n] = hi;
    ++l.n;
    return true;
  };
  const int first_extra = al ? nvb : 0, extras = kb + tb - first_extra;
  for (int blk = first_extra; blk < kb + tb; ++blk) {
    // an odd block out (MLA: the decoupled RoPE block) is loaded by both CTAs and each scores half of its
    // MMA steps, so both issue the same number of score MMAs per tile
    if (kSplitOddBlock && blk == kb + tb - 1 && (extras & 1) && out[0].n == out[1].n) {
      if (!put(0, blk, 0, 2) || !put(1, blk, 2, 4)) return false;
    } else if (!put(out[0].n <= out[1].n ? 0 : 1, blk, 0, 4)) {
      return false;
    }
  }
  // each CTA must score at least one block (its score buffer is exchanged every tile)
  for (int r = 0; r < 2; ++r) {
    BlockList& l = out[r];
    int ns = 0;
    l.ks0 = -1;
    l.steps = 0u;
    for (int i = 0; i < l.n; ++i) {
      if (l.qcol[i] < 0) {
        if (l.ks0 >= 0) return false;               // value-only blocks come first
        continue;
      }
      if (l.ks0 < 0) l.ks0 = i;
      for (int k4 = k4_lo[r][i]; k4 < k4_hi[r][i]; ++k4) l.steps |= 1u << (4 * (i - l.ks0) + k4);
      ++ns;
    }
    if (ns == 0 || l.n > MAXB) return false;
  }
  return true;
}

template <typename T_>
int launch(const CUtensorMap& tK, const CUtensorMap& tKt, const CUtensorMap& tV, const Args& a, int head_blocks,
           cudaStream_t st) {
  auto kern = latent_pair_kernel<T_>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) {
    cudaGetLastError();
    return XKV_ERR_LAUNCH;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(head_blocks * 2, a.batch, a.num_splits);
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kern, tK, tKt, tV, a) != cudaSuccess) {
    cudaGetLastError();
    return XKV_ERR_LAUNCH;
  }
  return cudaGetLastError() == cudaSuccess ? XKV_OK : XKV_ERR_LAUNCH;
}

// How many CTA pairs of this kernel the device holds at once.  Not simply SMs / 2: the two CTAs of a cluster
// must sit in one GPC, and a GPC with an odd number of usable SMs leaves one over.  Asked of the runtime once
// per device; without a device (planning on a CPU-only machine) SMs / 2.
int pair_slots() {
  constexpr int kMaxDevices = 64;
  static int cached[kMaxDevices] = {};
  const int fallback = device_sm_count() / 2;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return fallback;
  }
  if (dev >= 0 && dev < kMaxDevices && cached[dev] > 0) return cached[dev];
  auto kern = latent_pair_kernel<__nv_bfloat16>;
  int n = 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * device_sm_count(), 1, 1);
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess ||
      cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    return fallback;
  }
  if (dev >= 0 && dev < kMaxDevices) cached[dev] = n;
  return n;
}

}  // namespace

bool latent_pair_supported(const xkv_decode_params& p) {
  if (p.score_mode != XKV_SCORE_LATENT || p.value_mode != XKV_VALUE_LATENT) return false;
  if (p.flags & (XKV_FLAG_LOGITS_ONLY | XKV_FLAG_FORCE_GENERIC | XKV_FLAG_LATENT_MMA_SYNC)) return false;
  if (p.dtype != XKV_BF16 && p.dtype != XKV_F16) return false;
  if (p.logit_cap > 0.f || p.mask) return false;
  if (p.num_heads < 64) return false;      // fewer heads leave most MMA rows empty: the mma.sync kernel serves them
  if (p.batch > 65535) return false;       // the batch row is a grid y index
  if (p.k_rank % 64 != 0 || p.tail_dim % 64 != 0 || p.v_rank % 128 != 0 || p.v_rank > 512) return false;
  if (!aligned16(p.k) || !aligned16(p.v) || !stride_ok(p.k_sl) || !stride_ok(p.v_sl)) return false;
  if (p.batch > 1 && (!stride_ok(p.k_sb) || !stride_ok(p.v_sb))) return false;
  if (p.tail_dim > 0 && (!aligned16(p.k_tail) || !stride_ok(p.kt_sl) || (p.batch > 1 && !stride_ok(p.kt_sb)))) return false;
  BlockList bl[2];
  return make_lists(p, bl);
}

bool latent_pair_plan(const xkv_decode_params& p, LatentTcPlan* pl) {
  const int head_blocks = ceil_div(p.num_heads, 128);
  const int tiles = ceil_div(p.kv_len, T);
  const int rows = p.batch * head_blocks;
  const int slots = pair_slots();               // clusters of two CTAs the device holds at once
  int best_s = 1;
  int64_t best_cost = -1;
  const int max_s = tiles < 64 ? tiles : 64;
  for (int s = 1; s <= max_s; ++s) {
    const int64_t waves = ceil_div(rows * s, slots);
    const int64_t cost = waves * (ceil_div(tiles, s) + 6);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_s = s; }
  }
  pl->heads_per_cta = 128;
  pl->stages = STAGES;
  pl->smem_bytes = SMEM_BYTES;
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
  if (p.v_proj && p.vp_sb == 0 && batched_projection_fits(p.batch, p.v_rank)) {
    pl->off_olat = off;
    off += align_up((size_t)p.batch * p.num_heads * p.v_rank * sizeof(float), 256);
  }
  pl->total_bytes = off;
  return true;
}

int latent_pair_decode(const xkv_decode_params& p, const LatentTcPlan& pl, void* ws, cudaStream_t st) {
  char* w = static_cast<char*>(ws);
  const int dk = p.k_rank + p.tail_dim;
  CUtensorMap tK, tKt, tV;
  if (!encode_rows(&tK, p.dtype, p.k, p.k_rank, p.kv_len, p.batch, p.k_sl, p.k_sb)) return XKV_ERR_NO_DEVICE;
  if (p.tail_dim > 0) {
    if (!encode_rows(&tKt, p.dtype, p.k_tail, p.tail_dim, p.kv_len, p.batch, p.kt_sl, p.kt_sb)) return XKV_ERR_NO_DEVICE;
  } else {
    tKt = tK;
  }
  if (!aliased(p)) {
    if (!encode_rows(&tV, p.dtype, p.v, p.v_rank, p.kv_len, p.batch, p.v_sl, p.v_sb)) return XKV_ERR_NO_DEVICE;
  } else {
    tV = tK;
  }
  int* status = reinterpret_cast<int*>(w);
  sm100::clear_status_kernel<<<1, 64, 0, st>>>(status);
  void* qeff = w + pl.off_qeff;
  // queries that need no projection are read where they are when every row piece is 16-byte aligned
  const bool q_direct = p.k_proj == nullptr && aligned16(p.q) && p.q_sb % 8 == 0 && p.q_sh % 8 == 0 &&
                        (p.tail_dim == 0 || (aligned16(p.q_tail) && p.qt_sb % 8 == 0 && p.qt_sh % 8 == 0));
  // a projection shared by the batch is folded into the queries one matrix strip at a time (each matrix
  // element read once per strip of batch rows); per-batch projections go row by row
  int rc = q_direct ? XKV_OK
           : (p.k_proj && p.kp_sb == 0 && batched_projection_fits(p.batch, p.head_dim))
               ? launch_absorb_query_batched(p, qeff, dk, st)
               : launch_absorb_query_lowp(p, qeff, dk, st);
  if (rc != XKV_OK) return rc;
  // one split per row, no value projection, no log-sum-exp wanted: the kernel stores the result itself
  const bool out_direct = pl.num_splits == 1 && p.v_proj == nullptr && p.lse_out == nullptr && p.value_dim == p.v_rank &&
                          aligned16(p.out) && p.o_sb % 8 == 0 && p.o_sh % 8 == 0;
  Args a;
  a.q = p.q; a.q_tail = p.q_tail; a.q_sb = p.q_sb; a.q_sh = p.q_sh; a.qt_sb = p.qt_sb; a.qt_sh = p.qt_sh;
  a.q_cols = p.k_rank;
  a.out = out_direct ? p.out : nullptr; a.o_sb = p.o_sb; a.o_sh = p.o_sh;
  a.batch = p.batch; a.kv_len = p.kv_len; a.num_heads = p.num_heads; a.dk = dk;
  a.num_splits = pl.num_splits; a.tiles_per_row = pl.tiles;
  a.scale_log2 = p.sm_scale * 1.4426950408889634f;
  a.qeff = q_direct ? nullptr : qeff;
  a.partial_o = reinterpret_cast<float*>(w + pl.off_partial);
  a.lse = reinterpret_cast<float*>(w + pl.off_lse);
  a.rv = p.v_rank;
  a.status = status;
  a.kv_lens = p.kv_lens;
  if (!make_lists(p, a.bl)) return XKV_ERR_UNSUPPORTED;
  const int head_blocks = ceil_div(p.num_heads, 128);
  rc = p.dtype == XKV_BF16 ? launch<__nv_bfloat16>(tK, tKt, tV, a, head_blocks, st)
                           : launch<__half>(tK, tKt, tV, a, head_blocks, st);
  if (rc != XKV_OK) return rc;
  if (out_direct) return XKV_OK;
  if (pl.off_olat != 0 && pl.num_splits == 1 && !p.lse_out)   // one split: its normalised partial IS the latent output
    return launch_value_projection_batched(a.partial_o, p, st);
  if (pl.off_olat != 0 && !p.lse_out && value_projection_merges(p, pl.num_splits))   // a few splits: merged as the projection stages them
    return launch_value_projection_batched(a.partial_o, p, st, a.lse, pl.num_splits);
  if (pl.off_olat != 0) {
    // merge the splits in latent space (fp32), then apply the shared value projection batched over the rows
    float* o_lat = reinterpret_cast<float*>(w + pl.off_olat);
    rc = launch_merge(a.partial_o, a.lse, o_lat, XKV_F32, p.batch, p.num_heads, pl.num_splits, p.v_rank, p.v_rank, nullptr, 1,
                      0, 0, 0, 0, (int64_t)p.num_heads * p.v_rank, p.v_rank, st, 0, 0, p.lse_out, p.lse_sb);
    if (rc != XKV_OK) return rc;
    return launch_value_projection_batched(o_lat, p, st);
  }
  return launch_merge(a.partial_o, a.lse, p.out, p.dtype, p.batch, p.num_heads, pl.num_splits, p.v_rank, p.value_dim,
                      p.v_proj, p.v_proj ? p.v_proj_heads : 1, p.vp_sb, p.vp_sh, p.vp_sr, p.vp_sd, p.o_sb, p.o_sh, st, 0, 0,
                      p.lse_out, p.lse_sb);
}

}  // namespace xkv
