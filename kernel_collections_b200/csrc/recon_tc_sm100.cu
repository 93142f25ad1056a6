// Fused key reconstruction + RoPE + decode attention on the sm_100a tensor cores.
//
// Per 128-token tile of one batch row the keys of all KV heads are rebuilt as K = A_tile . B on
// tcgen05 (A: the latent tile, K-major; B: MN-major slices of the projection; fp32 accumulators in
// TMEM, two 128x256 buffers), rotated in registers straight out of TMEM, dotted with the query
// heads, pushed through an online softmax and multiplied into a dense V tile.  K never exists
// in shared or global memory.  One CTA per (KV split, batch row), twelve warps with fixed roles:
//
//   warp 0      TMA producer for the A / B operand ring (3 stages of 64 ranks)
//   warp 1      tcgen05.mma issuer (one elected thread), commits to mbarriers
//   warp 2      TMEM allocation, TMA producer for the V ring (2 slots of 128 tokens x 1 KV head)
//   warp 3      idle
//   warps 4-7   epilogue: tcgen05.ld, RoPE (angles reduced mod 2pi, sin/cos on the SFU), q-dot,
//               online softmax, P->smem
//   warps 8-11  P.V with mma.sync out of shared memory, running output / row-sum accumulators
//
// Every mbarrier wait is bounded: on expiry the kernel raises a shared abort flag, records where
// it gave up in the status words of the workspace, lets every role drain to the common exit,
// waits for copies in flight, frees its TMEM and returns.  No TMA load uses cluster multicast.
#include "sm100_common.cuh"

namespace xkv {
using namespace sm100;
namespace {

constexpr int TILE_M = 128;   // tokens per tile == TMEM lanes
constexpr int BK = 64;        // ranks per pipeline stage (one 128-byte swizzle row)
constexpr int D = 128;        // head dim
constexpr int KVH = 8;        // KV heads
constexpr int NCH = KVH / 2;  // chunks of two KV heads (256 accumulator columns)
constexpr int STAGES = 3;
constexpr int A_BYTES = TILE_M * BK * 2;       // 16 KB
constexpr int B_BOX = BK * 64 * 2;             // 8 KB: 64 n x 64 k
constexpr int B_BYTES = 4 * B_BOX;             // 32 KB: 256 n x 64 k
constexpr int STAGE_BYTES = A_BYTES + B_BYTES; // 48 KB
constexpr int V_SLOT = TILE_M * D * 2;         // 32 KB
constexpr int V_SLOTS = 2;
constexpr int P_PITCH = TILE_M * 2 + 16;       // bytes per head row of P (padded against bank conflicts)
constexpr int NTHREADS = 384;

constexpr int OFF_STAGE = 0;
constexpr int OFF_V = OFF_STAGE + STAGES * STAGE_BYTES;          // 147456
constexpr int OFF_Q = OFF_V + V_SLOTS * V_SLOT;                  // 212992
constexpr int Q_BYTES = 2 * 64 * 8 * 2 * 4;                      // 8192 (G <= 8)
constexpr int OFF_P = OFF_Q + Q_BYTES;                           // 221184
constexpr int P_BUF = 16 * P_PITCH;                              // 4352
constexpr int OFF_WMAX = OFF_P + 2 * P_BUF;                      // 229888
constexpr int OFF_ALPHA = OFF_WMAX + 2 * 4 * 16 * 4;             // +512
constexpr int OFF_M = OFF_ALPHA + 2 * 16 * 4;                    // +128
constexpr int OFF_BAR = OFF_M + 64 * 4;                          // +256
constexpr int NUM_BARS = 20;   // full[4] empty[4] tfull[2] tempty[2] vfull[2] vempty[2] pfull[2] pempty[2]
constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
constexpr int OFF_FREQ = OFF_MISC + 16;                          // 64 RoPE frequencies
constexpr int SMEM_USED = OFF_FREQ + 64 * 4;
constexpr int SMEM_BYTES = SMEM_USED + 1024;                     // + slack to align the base to 1024
static_assert(SMEM_BYTES <= 232448, "shared memory budget exceeded");


constexpr int MAX_LAYERS = 8;   // layers of one cross-layer group served by a single launch

// Tensor maps of one launch: the key latent is shared by all layers, projections and values are
// per layer.
struct TensorMaps {
  CUtensorMap a;
  CUtensorMap b[MAX_LAYERS];
  CUtensorMap v[MAX_LAYERS];
};

struct Args {
  int num_layers;
  int batch, kv_len, num_heads, rank;
  int num_splits, tiles_per_row;
  float q_scale;
  const void* q[MAX_LAYERS];
  int64_t q_sb, q_sh;
  const float* inv_freq; // 64 RoPE frequencies (device) or NULL -> theta
  float theta;
  int pos_offset;
  float* partial_o;      // [layer][batch][H][splits][128]
  float* lse;            // [layer][batch][H][splits]
  void* logits;
  int64_t lg_sb, lg_sh, lg_layer;   // logits[layer * lg_layer + b * lg_sb + h * lg_sh + token]
  int logits_f32;                   // logits are fp32 (the first pass of a two-pass decode) instead of T
  int* status;
  int b_batched;
  const int32_t* kv_lens;   // per-row lengths (ragged batches) or NULL
  int drop_load;            // fault-test build only: the producer announces one stage and does not load it
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers
#ifdef XKV_TC_PROFILE
// Debug build only: cycles spent in each kind of wait, summed over CTAs into status[8 + slot].
#define XKV_PROF_WAIT_L(slot, leader, expr)                                          \
  [&]() {                                                                            \
    const long long t0_ = clock64();                                                 \
    const bool r_ = (expr);                                                          \
    if (leader)                                                                      \
      atomicAdd(reinterpret_cast<unsigned long long*>(a.status + 8) + (slot),        \
                (unsigned long long)(clock64() - t0_));                              \
    return r_;                                                                       \
  }()
#else
#define XKV_PROF_WAIT_L(slot, leader, expr) (expr)
#endif
#define XKV_PROF_WAIT(slot, expr) XKV_PROF_WAIT_L(slot, true, expr)

// Barrier over the 128 epilogue threads that also agrees on the abort flag, so that either all of
// them leave or none does (a thread that left alone would strand the rest at the next barrier).
__device__ __forceinline__ bool epilogue_sync_aborted(volatile int* abort_flag) {
  const uint32_t mine = *abort_flag ? 1u : 0u;
  uint32_t any;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "barrier.cta.red.or.pred q, 1, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(any)
      : "r"(mine)
      : "memory");
  return any != 0;
}
// ---- thread-block-cluster helpers for the CTA-pair (cta_group::2) variant -----------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `local_addr` (an address in this CTA's shared window) in CTA `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA loads of the pair variant: the data lands in this CTA, the bytes are counted on the mbarrier
// of the leader CTA (`bar` is a shared::cluster address).  No multicast: each CTA fetches its own.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2,
                                                 uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                                 uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// sin / cos of an fp32 angle of any magnitude met here (|x| < 2^18): three-constant Cody-Waite
// reduction to [-pi, pi] (the first product is exact for |k| < 2^16), then the SFU
// approximations, whose absolute error on that interval is below 1e-6.
__device__ __forceinline__ void sincos_reduced(float x, float& sn, float& cs) {
  // round to nearest integer on the FMA pipe: |x / 2pi| < 2^22 here, so adding and removing
  // 1.5 * 2^23 leaves the rounded value (the conversion instruction shares the busy SFU pipe)
  const float k = __fadd_rn(__fadd_rn(x * 0.15915494309189535f, 12582912.0f), -12582912.0f);
  float r = fmaf(k, -6.28125f, x);
  r = fmaf(k, -1.9350051879882812e-3f, r);
  r = fmaf(k, -3.019916050561733e-7f, r);
  sn = __sinf(r);
  cs = __cosf(r);
}

// ---------------------------------------------------------------------------------------------
// PAIR: two CTAs of a cluster share every MMA (tcgen05 cta_group::2, M = 256): each loads its own
// 128-token latent tile and HALF of the B chunk (one KV head), the leader CTA issues the MMAs, and
// each CTA finds the keys of its own tokens for both KV heads in its own TMEM.  This halves the B
// bytes written to and read from shared memory, the unit that paces the 1-CTA kernel.  Everything
// after the accumulators (epilogue, V ring, P.V) is per CTA and unchanged.
// Two angles at a time on the packed fp32x2 pipe (Blackwell): same Cody-Waite steps, element-wise
// IEEE products and FMAs, then the SFU approximations per element.
__device__ __forceinline__ void sincos_reduced2(float2 x, float2& sn, float2& cs) {
  const float2 magic = make_float2(12582912.0f, 12582912.0f), nmagic = make_float2(-12582912.0f, -12582912.0f);
  const float2 k = __fadd2_rn(__ffma2_rn(x, make_float2(0.15915494309189535f, 0.15915494309189535f), magic), nmagic);
  float2 r = __ffma2_rn(k, make_float2(-6.28125f, -6.28125f), x);
  r = __ffma2_rn(k, make_float2(-1.9350051879882812e-3f, -1.9350051879882812e-3f), r);
  r = __ffma2_rn(k, make_float2(-3.019916050561733e-7f, -3.019916050561733e-7f), r);
  sn = make_float2(__sinf(r.x), __sinf(r.y));
  cs = make_float2(__cosf(r.x), __cosf(r.y));
}

template <typename T, int G, bool LOGITS_ONLY, bool PAIR>
__global__ void __launch_bounds__(NTHREADS, 1)
recon_tc_kernel(const __grid_constant__ TensorMaps maps, const Args a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The layer index varies fastest over the grid: the CTAs of one (split, batch row) that serve
  // the layers of a group are scheduled together and stream the same latent tiles, which are then
  // read from HBM once and served from L2 to the other layers.
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;           // 0 = leader of the pair
  const int unit = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int layer = unit % a.num_layers, split = unit / a.num_layers, b = blockIdx.y;
  const CUtensorMap* tmA = &maps.a;
  const CUtensorMap* tmB = &maps.b[layer];
  const CUtensorMap* tmV = &maps.v[layer];
  const int64_t row = (int64_t)layer * a.batch + b;   // row of the partial / lse buffers
  // tiles [range_begin, range_end) belong to this split; a pair interleaves them (leader even, peer
  // odd positions) and both CTAs run the same number of iterations, the peer possibly ending on
  // a phantom tile whose tokens are all masked
  const int row_len = a.kv_lens ? min(max(a.kv_lens[b], 0), a.kv_len) : a.kv_len;   // this row's length
  const int row_tiles = a.kv_lens ? (row_len + TILE_M - 1) / TILE_M : a.tiles_per_row;
  const int range_begin = (int)(((int64_t)split * row_tiles) / a.num_splits);
  const int range_end = (int)(((int64_t)(split + 1) * row_tiles) / a.num_splits);
  constexpr int TSTEP = PAIR ? 2 : 1;
  const int tile_begin = range_begin + (int)rank;
  const int tile_end = PAIR ? tile_begin + 2 * ((range_end - range_begin + 1) / 2) : range_end;
  const int out_split = PAIR ? split * 2 + (int)rank : split;       // slot of the partial / lse buffers
  const int out_splits = PAIR ? a.num_splits * 2 : a.num_splits;
  const int KB = a.rank / BK;
  constexpr int NSTAGE = PAIR ? 4 : STAGES;                          // the pair's stages are 32 KB
  constexpr int STAGE_SZ = PAIR ? A_BYTES + B_BYTES / 2 : STAGE_BYTES;

  const uint32_t bar0 = base + OFF_BAR;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (4 + s); };
  auto bar_tfull = [&](int i) { return bar0 + 8u * (8 + i); };
  auto bar_tempty = [&](int i) { return bar0 + 8u * (10 + i); };
  auto bar_vfull = [&](int i) { return bar0 + 8u * (12 + i); };
  auto bar_vempty = [&](int i) { return bar0 + 8u * (14 + i); };
  auto bar_pfull = [&](int i) { return bar0 + 8u * (16 + i); };
  auto bar_pempty = [&](int i) { return bar0 + 8u * (18 + i); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_MISC + 4);

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGE; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_tfull(i), 1);
      mbar_init(bar_tempty(i), PAIR ? 256 : 128);   // the leader also collects the peer's epilogue
      mbar_init(bar_vfull(i), 1);
      mbar_init(bar_vempty(i), 128);
      mbar_init(bar_pfull(i), 128);
      mbar_init(bar_pempty(i), 128);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 2) {
    if (PAIR) {   // both CTAs of the pair issue the allocation, same warp, same destination offset
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(base + OFF_MISC), "r"(512u) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(base + OFF_MISC), "r"(512u) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  if (threadIdx.x >= 128 && threadIdx.x < 256) {   // running maxima start at -inf
    float* m_s = reinterpret_cast<float*>(sm + OFF_M);
    if (threadIdx.x - 128 < 64) m_s[threadIdx.x - 128] = -CUDART_INF_F;
  }
  if (threadIdx.x >= 256 && threadIdx.x < 320) {
    const int j = threadIdx.x - 256;
    reinterpret_cast<float*>(sm + OFF_FREQ)[j] =
        a.inv_freq ? a.inv_freq[j] : 1.0f / powf(a.theta, (float)(2 * j) / (float)D);
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the peer's barriers exist before anything is signalled across CTAs
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
#ifdef XKV_TC_PROFILE
  const long long t_start_ = clock64();
  const uint64_t ns_start_ = global_ns();
#endif

  if (warp == 0) {
    // =========================== operand producer =============================================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const int bb = a.b_batched ? b : 0;
      for (int tile = tile_begin; tile < tile_end; tile += TSTEP) {
        for (int c = 0; c < NCH; ++c) {
          for (int kb = 0; kb < KB; ++kb) {
            if (!XKV_PROF_WAIT(0, mbar_wait(bar_empty(stage), phase ^ 1u, abort_flag))) {
              report(a.status, XKV_ERR_TIMEOUT, 0, tile, c, kb);
              goto producer_done;
            }
            const uint32_t sa = base + OFF_STAGE + stage * STAGE_SZ;
#ifdef XKV_FAULT_TEST
            if (!PAIR && a.drop_load && tile == tile_begin && c == 1 && kb == 0) {
              mbar_expect_tx(bar_full(stage), STAGE_BYTES);     // announced, never loaded: the consumer's wait runs out
              if (++stage == NSTAGE) { stage = 0; phase ^= 1u; }
              continue;
            }
#endif
            if (PAIR) {
              // bytes of both CTAs are counted on the leader's barrier, which the leader arms for both
              const uint32_t lead_full = map_to_cta(bar_full(stage), 0);
              if (rank == 0) mbar_expect_tx(bar_full(stage), 2 * STAGE_SZ);
              tma_load_3d_pair(sa, tmA, kb * BK, tile * TILE_M, b, lead_full);
#pragma unroll
              for (int i = 0; i < 2; ++i)   // this CTA's half of the chunk: KV head 2c + rank
                tma_load_4d_pair(sa + A_BYTES + i * B_BOX, tmB, i * 64, kb * BK, 2 * c + (int)rank, bb, lead_full);
            } else {
              mbar_expect_tx(bar_full(stage), STAGE_BYTES);
              tma_load_3d(sa, tmA, kb * BK, tile * TILE_M, b, bar_full(stage));
#pragma unroll
              for (int i = 0; i < 4; ++i)
                tma_load_4d(sa + A_BYTES + i * B_BOX, tmB, (i & 1) * 64, kb * BK, 2 * c + (i >> 1), bb, bar_full(stage));
            }
            if (++stage == NSTAGE) { stage = 0; phase ^= 1u; }
          }
        }
      }
    }
  producer_done:;
  } else if (warp == 1) {
    // =========================== MMA issuer ===================================================
    if (lane == 0 && rank == 0) {   // in a pair only the leader issues
      // instruction descriptor: fp32 accumulate, A K-major, B MN-major, N = 256, M = 128 (256 for a pair)
      const uint32_t idesc = (1u << 4) | (TypeTraits<T>::kFmt << 7) | (TypeTraits<T>::kFmt << 10) | (1u << 16) |
                             ((256u >> 3) << 17) | (((PAIR ? 256u : 128u) >> 4) << 24);
      int stage = 0, abuf = 0;
      uint32_t phase = 0, aphase = 0;
      // operand descriptors of stage 0, built once; the loops only add offsets
      const uint64_t da0 = smem_desc(base + OFF_STAGE, 16, 1024);
      const uint64_t db0 = smem_desc(base + OFF_STAGE + A_BYTES, B_BOX, 1024);
      for (int tile = tile_begin; tile < tile_end; tile += TSTEP) {
        for (int c = 0; c < NCH; ++c) {
          if (!XKV_PROF_WAIT(1, mbar_wait(bar_tempty(abuf), aphase ^ 1u, abort_flag))) {
            report(a.status, XKV_ERR_TIMEOUT, 1, tile, c, -1);
            goto mma_done;
          }
          tc_fence_after();
          const uint32_t tacc = tmem_base + (uint32_t)abuf * 256u;
          for (int kb = 0; kb < KB; ++kb) {
            if (!XKV_PROF_WAIT(2, mbar_wait(bar_full(stage), phase, abort_flag))) {
              report(a.status, XKV_ERR_TIMEOUT, 1, tile, c, kb);
              goto mma_done;
            }
            tc_fence_after();
            const uint64_t da_st = desc_advance(da0, (uint32_t)(stage * STAGE_SZ));
            const uint64_t db_st = desc_advance(db0, (uint32_t)(stage * STAGE_SZ));
#pragma unroll
            for (int k4 = 0; k4 < BK / 16; ++k4) {
              const uint64_t da = desc_advance(da_st, k4 * 32);
              const uint64_t db = desc_advance(db_st, k4 * 2048);
              if (PAIR) tc_mma_pair(tacc, da, db, idesc, (kb | k4) != 0 ? 1u : 0u);
              else tc_mma(tacc, da, db, idesc, (kb | k4) != 0 ? 1u : 0u);
            }
            if (PAIR) {   // free the stage in both CTAs (two plain commits, one per CTA)
              tc_commit_pair(map_to_cta(bar_empty(stage), 0));
              tc_commit_pair(map_to_cta(bar_empty(stage), 1));
            } else {
              tc_commit(bar_empty(stage));
            }
            if (++stage == NSTAGE) { stage = 0; phase ^= 1u; }
          }
          if (PAIR) {
            tc_commit_pair(map_to_cta(bar_tfull(abuf), 0));
            tc_commit_pair(map_to_cta(bar_tfull(abuf), 1));
          } else {
            tc_commit(bar_tfull(abuf));
          }
          abuf ^= 1;
          if (abuf == 0) aphase ^= 1u;
        }
      }
    }
  mma_done:;
  } else if (warp == 2) {
    // =========================== V producer ===================================================
    if (!LOGITS_ONLY && lane == 0) {
      int slot = 0;
      uint32_t ph = 0;
      for (int tile = tile_begin; tile < tile_end; tile += TSTEP) {
        for (int kvh = 0; kvh < KVH; ++kvh) {
          if (!XKV_PROF_WAIT(3, mbar_wait(bar_vempty(slot), ph ^ 1u, abort_flag))) {
            report(a.status, XKV_ERR_TIMEOUT, 2, tile, kvh, -1);
            goto vprod_done;
          }
          mbar_expect_tx(bar_vfull(slot), V_SLOT);
          const uint32_t sv = base + OFF_V + slot * V_SLOT;
          tma_load_4d(sv, tmV, 0, kvh, tile * TILE_M, b, bar_vfull(slot));
          tma_load_4d(sv + V_SLOT / 2, tmV, 64, kvh, tile * TILE_M, b, bar_vfull(slot));
          if (++slot == V_SLOTS) { slot = 0; ph ^= 1u; }
        }
      }
    }
  vprod_done:;
  } else if (warp >= 4 && warp < 8) {
    // =========================== epilogue =====================================================
    const int et = threadIdx.x - 128;
    const int ew = et >> 5;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(ew * 32) << 16);
    float* q_s = reinterpret_cast<float*>(sm + OFF_Q);
    float* wmax_s = reinterpret_cast<float*>(sm + OFF_WMAX);
    float* alpha_s = reinterpret_cast<float*>(sm + OFF_ALPHA);
    float* m_s = reinterpret_cast<float*>(sm + OFF_M);
    const T* qg = static_cast<const T*>(a.q[layer]) + (int64_t)b * a.q_sb;
    const float* freq_s = reinterpret_cast<const float*>(sm + OFF_FREQ);
    int abuf = 0, pbuf = 0, par = 0;
    uint32_t aphase = 0, pphase = 0;
    // The chunk's queries (2 KV heads x G heads x 128 dims) are fetched one chunk ahead into
    // registers, 8 elements per 128-bit load, so their L2 latency hides under the previous chunk.
    constexpr int QV = (2 * G * D) / (128 * 8);
    uint4 qpre[QV];
    auto q_fetch = [&](int c) {
#pragma unroll
      for (int v = 0; v < QV; ++v) {
        const int idx = (v * 128 + et) * 8;
        const int hh = idx / (G * D), g = (idx / D) % G, d = idx % D;
        qpre[v] = *reinterpret_cast<const uint4*>(qg + (int64_t)((2 * c + hh) * G + g) * a.q_sh + d);
      }
    };
    q_fetch(0);
    for (int tile = tile_begin; tile < tile_end; tile += TSTEP) {
      const int tok = tile * TILE_M + et;
      const bool valid = tok < row_len && tile < range_end;   // (a pair's peer may end on a phantom tile)
      const float pos_f = (float)(a.pos_offset + tok);
      for (int c = 0; c < NCH; ++c) {
        // ---- stage this chunk's queries: q_s[hh][j][g][{j, j+64}] = q * scale -----------------
        if (epilogue_sync_aborted(abort_flag)) goto epi_done;
#pragma unroll
        for (int v = 0; v < QV; ++v) {
          const int idx = (v * 128 + et) * 8;
          const int hh = idx / (G * D), g = (idx / D) % G, d0 = idx % D;
          const T* e8 = reinterpret_cast<const T*>(&qpre[v]);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int d = d0 + e;
            // pairs of frequencies side by side: [hh][j / 2][g][{x_j, x_j+1, y_j, y_j+1}], x = dim j, y = dim j + 64
            const int j = d & 63;
            q_s[((hh * 32 + (j >> 1)) * G + g) * 4 + (d >> 6) * 2 + (j & 1)] = TypeTraits<T>::to_f(e8[e]) * a.q_scale;
          }
        }
        q_fetch((c + 1) % NCH);
        float m_old[2 * G];
        if (!LOGITS_ONLY) {
#pragma unroll
          for (int i = 0; i < 2 * G; ++i) m_old[i] = m_s[c * 2 * G + i];
        }
        if (epilogue_sync_aborted(abort_flag)) goto epi_done;
        if (!XKV_PROF_WAIT_L(4, et == 0, mbar_wait(bar_tfull(abuf), aphase, abort_flag))) report(a.status, XKV_ERR_TIMEOUT, 4, tile, c, 0);
        tc_fence_after();

        // logits accumulate on the packed fp32x2 pipe: lane .x holds the even frequencies, .y the odd
        float2 s2[2 * G];
#pragma unroll
        for (int i = 0; i < 2 * G; ++i) s2[i] = make_float2(0.f, 0.f);
        const float2 pos2 = make_float2(pos_f, pos_f);
#pragma unroll 1
        for (int jb = 0; jb < 4; ++jb) {
          // rotation of this token for frequencies jb*16 .. jb*16+15, shared by both KV heads
          float2 cs[8], sn[8], nsn[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float2 f2 = *reinterpret_cast<const float2*>(freq_s + jb * 16 + 2 * i);
            sincos_reduced2(__fmul2_rn(pos2, f2), sn[i], cs[i]);
            nsn[i] = make_float2(-sn[i].x, -sn[i].y);
          }
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t x0[16], x1[16];
            const uint32_t col = (uint32_t)abuf * 256u + hh * 128 + jb * 16;
            tmem_ld16(lane_addr + col, x0);
            tmem_ld16(lane_addr + col + 64, x1);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float2 k0 = make_float2(__uint_as_float(x0[2 * i]), __uint_as_float(x0[2 * i + 1]));
              const float2 k1 = make_float2(__uint_as_float(x1[2 * i]), __uint_as_float(x1[2 * i + 1]));
              const float2 r0 = __ffma2_rn(k0, cs[i], __fmul2_rn(k1, nsn[i]));
              const float2 r1 = __ffma2_rn(k1, cs[i], __fmul2_rn(k0, sn[i]));
              const float4* qp = reinterpret_cast<const float4*>(q_s + ((hh * 32 + jb * 8 + i) * G) * 4);
#pragma unroll
              for (int g = 0; g < G; ++g) {
                const float4 qq = qp[g];
                s2[hh * G + g] = __ffma2_rn(make_float2(qq.x, qq.y), r0,
                                            __ffma2_rn(make_float2(qq.z, qq.w), r1, s2[hh * G + g]));
              }
            }
          }
        }
        float s[2 * G];
#pragma unroll
        for (int i = 0; i < 2 * G; ++i) s[i] = s2[i].x + s2[i].y;
        tc_fence_before();
        if (PAIR && rank != 0) mbar_arrive_cluster(map_to_cta(bar_tempty(abuf), 0));   // the leader issues the MMAs
        else mbar_arrive(bar_tempty(abuf));
        abuf ^= 1;
        if (abuf == 0) aphase ^= 1u;

        if (LOGITS_ONLY) {
          if (valid) {
            const int64_t off = (int64_t)layer * a.lg_layer + (int64_t)b * a.lg_sb + tok;
            if (a.logits_f32) {
              float* lg = static_cast<float*>(a.logits) + off;
#pragma unroll
              for (int i = 0; i < 2 * G; ++i) lg[(int64_t)(2 * c * G + i) * a.lg_sh] = s[i];
            } else {
              T* lg = static_cast<T*>(a.logits) + off;
#pragma unroll
              for (int i = 0; i < 2 * G; ++i) lg[(int64_t)(2 * c * G + i) * a.lg_sh] = TypeTraits<T>::from_f(s[i]);
            }
          }
        } else {
          // ---- online softmax over the tile, per head -------------------------------------------
#pragma unroll
          for (int i = 0; i < 2 * G; ++i) {
            if (!valid) s[i] = -CUDART_INF_F;
            float wm = s[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, o));
            if (lane == 0) wmax_s[(par * 4 + ew) * 16 + i] = wm;
          }
          if (epilogue_sync_aborted(abort_flag)) goto epi_done;
          float m_new[2 * G], m_use[2 * G];
#pragma unroll
          for (int i = 0; i < 2 * G; ++i) {
            float mx = m_old[i];
#pragma unroll
            for (int w = 0; w < 4; ++w) mx = fmaxf(mx, wmax_s[(par * 4 + w) * 16 + i]);
            m_new[i] = mx;
            if (mx == -CUDART_INF_F) mx = 0.f;   // nothing seen yet (phantom tile): keep exp2 finite
            m_use[i] = mx;
          }
          par ^= 1;
          if (!XKV_PROF_WAIT_L(5, et == 0, mbar_wait(bar_pempty(pbuf), pphase ^ 1u, abort_flag))) report(a.status, XKV_ERR_TIMEOUT, 4, tile, c, 1);
          T* p_s = reinterpret_cast<T*>(sm + OFF_P + pbuf * P_BUF);
#pragma unroll
          for (int i = 0; i < 2 * G; ++i)
            p_s[i * (P_PITCH / 2) + et] = TypeTraits<T>::from_f(exp2f(s[i] - m_use[i]));
          if (et == 0) {
#pragma unroll
            for (int i = 0; i < 2 * G; ++i) {
              alpha_s[pbuf * 16 + i] = exp2f(m_old[i] - m_use[i]);
              m_s[c * 2 * G + i] = m_new[i];
            }
          }
          mbar_arrive(bar_pfull(pbuf));
          pbuf ^= 1;
          if (pbuf == 0) pphase ^= 1u;
        }
      }
    }
  epi_done:;
  } else if (warp >= 8) {
    // =========================== P.V ==========================================================
    if (!LOGITS_ONLY) {
      const int pw = warp - 8;
      const int g = lane >> 2, t = lane & 3;
      float acc[KVH][2][4];
      float lacc[KVH][4];
#pragma unroll
      for (int k = 0; k < KVH; ++k) {
#pragma unroll
        for (int i = 0; i < 4; ++i) { acc[k][0][i] = 0.f; acc[k][1][i] = 0.f; lacc[k][i] = 0.f; }
      }
      const float* alpha_s = reinterpret_cast<const float*>(sm + OFF_ALPHA);
      const float* m_s = reinterpret_cast<const float*>(sm + OFF_M);
      const uint32_t ones[4] = {TypeTraits<T>::ones2(), TypeTraits<T>::ones2(), TypeTraits<T>::ones2(),
                                TypeTraits<T>::ones2()};
      int slot = 0, pbuf = 0;
      uint32_t vph = 0, pph = 0;
      bool alive = true;
      for (int tile = tile_begin; tile < tile_end && alive; tile += TSTEP) {
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          bool ok = XKV_PROF_WAIT_L(6, threadIdx.x == 256, mbar_wait(bar_pfull(pbuf), pph, abort_flag));
          if (!__all_sync(0xffffffffu, ok)) {
            if (lane == 0) report(a.status, XKV_ERR_TIMEOUT, 8, tile, c, 0);
            alive = false;
            break;
          }
          const uint32_t p_base = base + OFF_P + pbuf * P_BUF;
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int kvh = 2 * c + hh;
            ok = XKV_PROF_WAIT_L(7, threadIdx.x == 256, mbar_wait(bar_vfull(slot), vph, abort_flag));
            if (!__all_sync(0xffffffffu, ok)) {
              if (lane == 0) report(a.status, XKV_ERR_TIMEOUT, 8, tile, c, 1 + hh);
              alive = false;
              break;
            }
            const float al0 = (2 * t < G) ? alpha_s[pbuf * 16 + hh * G + 2 * t] : 1.f;
            const float al1 = (2 * t + 1 < G) ? alpha_s[pbuf * 16 + hh * G + 2 * t + 1] : 1.f;
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
              acc[kvh][mt][0] *= al0; acc[kvh][mt][1] *= al1;
              acc[kvh][mt][2] *= al0; acc[kvh][mt][3] *= al1;
            }
            lacc[kvh][0] *= al0; lacc[kvh][1] *= al1; lacc[kvh][2] *= al0; lacc[kvh][3] *= al1;
            const uint32_t v_base = base + OFF_V + slot * V_SLOT;
            // ldmatrix row of this lane: matrix mi = lane / 8, row r = lane % 8
            const int mi = lane >> 3, r = lane & 7;
            if (a.kv_lens != nullptr && (tile + 1) * TILE_M > row_len) {
              // Ragged batch, last tile of the row: cache rows past the row's own length are outside
              // the call (they may hold anything, NaN included, and 0 * NaN is NaN).  This warp zeroes
              // the 32 value columns it reads itself, so no other warp has to wait for it.
              const int first = max(row_len - tile * TILE_M, 0);
              for (int idx = lane; idx < (TILE_M - first) * 4; idx += 32) {
                const int token = first + (idx >> 2), dim = pw * 32 + (idx & 3) * 8;
                const uint32_t za = v_base + (dim >> 6) * (V_SLOT / 2) + token * 128 +
                                    ((((dim & 63) >> 3) ^ (token & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(za), "r"(0u) : "memory");
              }
              __syncwarp();
            }
#pragma unroll
            for (int ks = 0; ks < TILE_M / 16; ++ks) {
              uint32_t b0 = 0, b1 = 0;
              if (g < G) {
                const uint32_t pa = p_base + (hh * G + g) * P_PITCH + (ks * 16 + 2 * t) * 2;
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(b0) : "r"(pa));
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(b1) : "r"(pa + 16));
              }
#pragma unroll
              for (int mt = 0; mt < 2; ++mt) {
                const int token = ks * 16 + (mi >> 1) * 8 + r;
                const int dim = pw * 32 + mt * 16 + (mi & 1) * 8;
                const uint32_t va = v_base + (dim >> 6) * (V_SLOT / 2) + token * 128 +
                                    ((((dim & 63) >> 3) ^ (token & 7)) << 4);
                uint32_t af[4];
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(af[0]), "=r"(af[1]), "=r"(af[2]), "=r"(af[3])
                             : "r"(va));
                TypeTraits<T>::mma(acc[kvh][mt], af, b0, b1);
              }
              TypeTraits<T>::mma(lacc[kvh], ones, b0, b1);
            }
            // The slot is refilled by TMA (async proxy) while it was read with ldmatrix (generic
            // proxy): a cross-proxy fence must separate this warp's reads from the release,
            // otherwise a refill can land under reads that are still in flight.
            __syncwarp();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(bar_vempty(slot));
            if (++slot == V_SLOTS) { slot = 0; vph ^= 1u; }
          }
          if (!alive) break;
          mbar_arrive(bar_pempty(pbuf));
          pbuf ^= 1;
          if (pbuf == 0) pph ^= 1u;
        }
      }
      if (alive && range_end <= range_begin) {
        // a split without tokens (short row of a ragged batch): publish an empty partial
        const int H = KVH * G;
        for (int h = lane; h < H; h += 32) {
          if (pw == 0) a.lse[(row * H + h) * out_splits + out_split] = -CUDART_INF_F;
          float* po = a.partial_o + ((row * H + h) * out_splits + out_split) * D + pw * 32;
          for (int d = 0; d < 32; ++d) po[d] = 0.f;
        }
      }
      if (alive && range_end > range_begin) {
        // normalised partial output and log-sum-exp of this split
        const int H = KVH * G;
#pragma unroll
        for (int kvh = 0; kvh < KVH; ++kvh) {
#pragma unroll
          for (int n = 0; n < 2; ++n) {
            const int hd = 2 * t + n;
            if (hd < G) {
              const int h = kvh * G + hd;
              const float l = lacc[kvh][n];
              const float inv = l > 0.f ? 1.f / l : 0.f;
              float* po = a.partial_o + ((row * H + h) * out_splits + out_split) * D;
#pragma unroll
              for (int mt = 0; mt < 2; ++mt) {
                const int dim = pw * 32 + mt * 16 + g;
                po[dim] = acc[kvh][mt][n] * inv;
                po[dim + 8] = acc[kvh][mt][2 + n] * inv;
              }
              if (pw == 0 && g == 0)
                a.lse[(row * H + h) * out_splits + out_split] =
                    l > 0.f ? (m_s[h] + log2f(l)) * 0.6931471805599453f : -CUDART_INF_F;
            }
          }
        }
      }
    }
  }

  // =========================== common exit =====================================================
#ifdef XKV_TC_PROFILE
  if (threadIdx.x == 128)   // epilogue leader: time from start until the epilogue has finished
    atomicAdd(reinterpret_cast<unsigned long long*>(a.status + 8) + 8, (unsigned long long)(clock64() - t_start_));
  if (threadIdx.x == 32)    // MMA issuer
    atomicAdd(reinterpret_cast<unsigned long long*>(a.status + 8) + 9, (unsigned long long)(clock64() - t_start_));
  if (threadIdx.x == 256)   // P.V leader
    atomicAdd(reinterpret_cast<unsigned long long*>(a.status + 8) + 10, (unsigned long long)(clock64() - t_start_));
  if (threadIdx.x == 0) {   // SM cycles and nanoseconds of this CTA: their ratio is the SM clock under load
    atomicAdd(reinterpret_cast<unsigned long long*>(a.status + 8) + 11, (unsigned long long)(clock64() - t_start_));
    atomicAdd(reinterpret_cast<unsigned long long*>(a.status + 8) + 12, (unsigned long long)(global_ns() - ns_start_));
  }
#endif
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // give copies and MMAs that may still be in flight time to land before the CTA's shared
    // memory and TMEM are released
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (PAIR) {
    // neither CTA leaves (or frees TMEM) while the other may still signal its barriers or have MMAs
    // reading its shared memory
    tc_fence_before();
    cluster_sync_all();
  }
  if (warp == 2) {
    tc_fence_after();
    if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

template <typename T, int G, bool LO, bool PAIR>
int launch_variant(const TensorMaps& maps, const Args& args, cudaStream_t st) {
  auto kern = recon_tc_kernel<T, G, LO, PAIR>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) {
    cudaGetLastError();
    return XKV_ERR_LAUNCH;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(args.num_splits * args.num_layers * (PAIR ? 2 : 1), args.batch);
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = PAIR ? 2 : 1;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kern, maps, args) != cudaSuccess) {
    cudaGetLastError();
    return XKV_ERR_LAUNCH;
  }
  return cudaGetLastError() == cudaSuccess ? XKV_OK : XKV_ERR_LAUNCH;
}

template <typename T, int G, bool LO>
int launch(const TensorMaps& maps, const Args& args, bool pair, cudaStream_t st) {
  return pair ? launch_variant<T, G, LO, true>(maps, args, st) : launch_variant<T, G, LO, false>(maps, args, st);
}

}  // namespace

bool recon_tc_supported(const xkv_decode_params& p) {
  if (p.score_mode != XKV_SCORE_RECON_ROPE) return false;
  if (p.dtype != XKV_BF16 && p.dtype != XKV_F16) return false;
  if (p.head_dim != D || p.num_kv_heads != KVH || p.k_proj_heads != KVH) return false;
  const int G = p.num_heads / p.num_kv_heads;
  if (G != 4 && G != 8) return false;
  if (p.k_rank < BK || p.k_rank % BK != 0) return false;
  if (p.tail_dim != 0 || p.logit_cap > 0.f) return false;
  if (p.mask) return false;   // additive masks run on the portable kernels
  if (p.rope_table) return false;   // caller-made tables go through the portable kernel
  if (p.q_sh % 8 != 0 || (p.batch > 1 && p.q_sb % 8 != 0)) return false;
  if (p.kp_sd != 1 || !aligned16(p.k) || !aligned16(p.k_proj) || !aligned16(p.q)) return false;
  if (!stride_ok(p.k_sl) || (p.batch > 1 && !stride_ok(p.k_sb))) return false;
  if (!stride_ok(p.kp_sr) || !stride_ok(p.kp_sh)) return false;
  if (p.kp_sb != 0 && !stride_ok(p.kp_sb)) return false;
  if (p.q_sh < D) return false;
  if (!(p.flags & XKV_FLAG_LOGITS_ONLY)) {
    if (p.value_mode != XKV_VALUE_DENSE || p.value_dim != D) return false;
    if (!aligned16(p.v) || !stride_ok(p.v_sl) || !stride_ok(p.v_sh)) return false;
    if (p.batch > 1 && !stride_ok(p.v_sb)) return false;
  }
  return true;
}

// Split count for `rows` independent (layer, batch row) streams of `tiles` tiles each.
static int choose_splits(int rows, int tiles) {
  const int sms = device_sm_count();
  int best_s = 1;
  int64_t best_cost = -1;
  const int max_s = tiles < 64 ? tiles : 64;
  for (int s = 1; s <= max_s; ++s) {
    const int64_t waves = ceil_div(rows * s, sms);
    const int64_t cost = waves * (ceil_div(tiles, s) + 1);   // + one tile of set-up and drain per CTA
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_s = s; }
  }
  return best_s;
}

// Whether the CTA-pair (cta_group::2) variant serves a call.  Two CTAs sharing each MMA halve the bytes
// of B that every SM pulls through shared memory; that pays once the rank contraction dominates
// (measured: rank 1024, 4 % faster; rank 512, 10 % slower because the leader then waits for two
// epilogues per accumulator) and there are enough tiles to fill the 74 pair slots.  The caller can
// pin either variant with XKV_FLAG_RECON_PAIR / XKV_FLAG_RECON_SINGLE_CTA.
static bool want_pair(const xkv_decode_params& p, int tiles, int rows) {
  if (p.flags & XKV_FLAG_RECON_SINGLE_CTA) return false;
  if (tiles < 2) return false;
  if (p.flags & XKV_FLAG_RECON_PAIR) return true;
  return p.k_rank >= 1024 && (int64_t)rows * tiles >= 8 * (int64_t)device_sm_count();
}

static bool plan_layers(const xkv_decode_params& p, int num_layers, ReconTcPlan* pl) {
  const int tiles = ceil_div(p.kv_len, TILE_M);
  const int rows = p.batch * num_layers;
  pl->pair = want_pair(p, tiles, rows) ? 1 : 0;
  if (pl->pair) {
    // splits are served by pairs of CTAs: SMs / 2 slots, each slot works through ceil(tiles / 2) rounds
    const int slots = device_sm_count() / 2;
    int best_s = 1;
    int64_t best_cost = -1;
    const int max_s = tiles / 2 < 64 ? tiles / 2 : 64;
    for (int s = 1; s <= max_s; ++s) {
      const int64_t waves = ceil_div(rows * s, slots);
      // + one round of set-up, pipeline fill and drain per CTA pair (measured on batch 128 x 131072 tokens: 8 rounds
      // per pair, which the count alone prefers, run 2.7 % slower than 128 rounds per pair)
      const int64_t cost = waves * (ceil_div(ceil_div(tiles, s), 2) + 1);
      if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_s = s; }
    }
    pl->num_splits = best_s;
  } else {
    pl->num_splits = choose_splits(rows, tiles);
  }
  pl->tiles_per_split = tiles;   // tiles per batch row; the kernel cuts [s*T/S, (s+1)*T/S)
  const int out_splits = pl->num_splits * (pl->pair ? 2 : 1);
  size_t off = 256;              // status words
  pl->off_partial = off;
  const bool lo = (p.flags & XKV_FLAG_LOGITS_ONLY) != 0;
  const size_t nrows = (size_t)num_layers * p.batch * p.num_heads * out_splits;
  if (!lo) off += align_up(nrows * D * sizeof(float), 256);
  pl->off_lse = off;
  if (!lo) off += align_up(nrows * sizeof(float), 256);
  pl->total_bytes = off;
  return true;
}

bool recon_tc_plan(const xkv_decode_params& p, ReconTcPlan* pl) { return plan_layers(p, 1, pl); }

bool recon_tc_group_supported(const xkv_decode_params* layers, int n) {
  if (n < 1 || n > MAX_LAYERS) return false;
  for (int i = 0; i < n; ++i) {
    const xkv_decode_params &a = layers[0], &b = layers[i];
    if (!recon_tc_supported(b) || (b.flags & (XKV_FLAG_LOGITS_ONLY | XKV_FLAG_FORCE_GENERIC))) return false;
    if (a.q_sb != b.q_sb || a.q_sh != b.q_sh || a.sm_scale != b.sm_scale || a.theta != b.theta ||
        a.pos_offset != b.pos_offset || a.inv_freq != b.inv_freq || a.k != b.k || a.k_sb != b.k_sb ||
        a.k_sl != b.k_sl || (a.kp_sb != 0) != (b.kp_sb != 0) || a.kv_lens != b.kv_lens)
      return false;
  }
  return true;
}

bool recon_tc_group_plan(const xkv_decode_params* layers, int n, ReconTcPlan* pl) {
  return plan_layers(layers[0], n, pl);
}

static bool encode_b(CUtensorMap* m, const xkv_decode_params& p, int b_batched) {
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)p.k_rank, (cuuint64_t)KVH, (cuuint64_t)(b_batched ? p.batch : 1)};
  const int64_t sb = b_batched ? p.kp_sb : (int64_t)KVH * p.k_rank * D * 4;
  const cuuint64_t strides[3] = {(cuuint64_t)p.kp_sr * 2, (cuuint64_t)p.kp_sh * 2, (cuuint64_t)sb * 2};
  const cuuint32_t box[4] = {64, BK, 1, 1};
  return encode_tiled_16bit(m, p.dtype, 4, p.k_proj, dims, strides, box);
}

static bool encode_v(CUtensorMap* m, const xkv_decode_params& p) {
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)KVH, (cuuint64_t)p.kv_len, (cuuint64_t)p.batch};
  const int64_t sb = p.batch > 1 ? p.v_sb : (int64_t)p.kv_len * KVH * D * 4;
  const cuuint64_t strides[3] = {(cuuint64_t)p.v_sh * 2, (cuuint64_t)p.v_sl * 2, (cuuint64_t)sb * 2};
  const cuuint32_t box[4] = {64, 1, TILE_M, 1};
  return encode_tiled_16bit(m, p.dtype, 4, p.v, dims, strides, box);
}

int recon_tc_group_decode(const xkv_decode_params* layers, int n, const ReconTcPlan& pl, void* ws,
                          cudaStream_t st, const LogitsSink* sink) {
  const xkv_decode_params& p = layers[0];
  char* w = static_cast<char*>(ws);
  if (!aligned16(w)) return XKV_ERR_ALIGN;
  const bool lo = sink != nullptr || (p.flags & XKV_FLAG_LOGITS_ONLY) != 0;
  const int G = p.num_heads / p.num_kv_heads;

  TensorMaps maps;
  {
    const cuuint64_t dims[3] = {(cuuint64_t)p.k_rank, (cuuint64_t)p.kv_len, (cuuint64_t)p.batch};
    const int64_t sb = p.batch > 1 ? p.k_sb : (int64_t)p.kv_len * p.k_sl;
    const cuuint64_t strides[2] = {(cuuint64_t)p.k_sl * 2, (cuuint64_t)sb * 2};
    const cuuint32_t box[3] = {BK, TILE_M, 1};
    if (!encode_tiled_16bit(&maps.a, p.dtype, 3, p.k, dims, strides, box)) return XKV_ERR_NO_DEVICE;
  }
  const int b_batched = (p.kp_sb != 0 && p.batch > 1) ? 1 : 0;
  for (int i = 0; i < MAX_LAYERS; ++i) {
    const xkv_decode_params& li = layers[i < n ? i : 0];
    if (i < n) {
      if (!encode_b(&maps.b[i], li, b_batched)) return XKV_ERR_NO_DEVICE;
      if (!lo) {
        if (!encode_v(&maps.v[i], li)) return XKV_ERR_NO_DEVICE;
      } else {
        maps.v[i] = maps.a;
      }
    } else {
      maps.b[i] = maps.b[0];
      maps.v[i] = maps.v[0];
    }
  }

  int* status = reinterpret_cast<int*>(w);
  clear_status_kernel<<<1, 64, 0, st>>>(status);

  Args a;
  a.num_layers = n;
  a.batch = p.batch; a.kv_len = p.kv_len; a.num_heads = p.num_heads; a.rank = p.k_rank;
  a.num_splits = pl.num_splits; a.tiles_per_row = pl.tiles_per_split;
  a.q_scale = lo ? p.sm_scale : p.sm_scale * 1.4426950408889634f;
  for (int i = 0; i < MAX_LAYERS; ++i) a.q[i] = layers[i < n ? i : 0].q;
  a.q_sb = p.q_sb; a.q_sh = p.q_sh;
  a.inv_freq = p.inv_freq; a.theta = p.theta; a.pos_offset = p.pos_offset;
  a.partial_o = reinterpret_cast<float*>(w + pl.off_partial);
  a.lse = reinterpret_cast<float*>(w + pl.off_lse);
  a.logits = p.logits; a.lg_sb = p.lg_sb; a.lg_sh = p.lg_sh; a.lg_layer = 0; a.logits_f32 = 0;
  if (sink) {
    a.logits = sink->ptr; a.lg_sb = sink->sb; a.lg_sh = sink->sh; a.lg_layer = sink->layer; a.logits_f32 = 1;
  }
  a.status = status;
  a.b_batched = b_batched;
  a.kv_lens = p.kv_lens;
  a.drop_load = 0;
#ifdef XKV_FAULT_TEST
  a.drop_load = (p.flags & XKV_FLAG_TEST_DROP_LOAD) ? 1 : 0;
#endif

  int rc;
#define XKV_TC(T, GG) rc = lo ? launch<T, GG, true>(maps, a, pl.pair != 0, st) : launch<T, GG, false>(maps, a, pl.pair != 0, st)
  if (p.dtype == XKV_BF16) {
    if (G == 4) { XKV_TC(__nv_bfloat16, 4); } else { XKV_TC(__nv_bfloat16, 8); }
  } else {
    if (G == 4) { XKV_TC(__half, 4); } else { XKV_TC(__half, 8); }
  }
#undef XKV_TC
  if (rc != XKV_OK) return rc;
  if (lo) return XKV_OK;
  const int out_splits = pl.num_splits * (pl.pair ? 2 : 1);
  const size_t layer_rows = (size_t)p.batch * p.num_heads * out_splits;
  for (int i = 0; i < n; ++i) {
    rc = launch_merge(a.partial_o + i * layer_rows * D, a.lse + i * layer_rows, layers[i].out, p.dtype, p.batch,
                      p.num_heads, out_splits, D, D, nullptr, 1, 0, 0, 0, 0, layers[i].o_sb, layers[i].o_sh, st, 0, 0, layers[i].lse_out,
                      layers[i].lse_sb);
    if (rc != XKV_OK) return rc;
  }
  return XKV_OK;
}

int recon_tc_decode(const xkv_decode_params& p, const ReconTcPlan& pl, void* ws, cudaStream_t st) {
  return recon_tc_group_decode(&p, 1, pl, ws, st, nullptr);
}

// First pass of the two-pass decode: logits only, so the value side of the blocks is not looked at.
bool recon_tc_logits_supported(const xkv_decode_params* layers, int n) {
  if (n < 1 || n > MAX_LAYERS) return false;
  for (int i = 0; i < n; ++i) {
    xkv_decode_params t = layers[i];
    t.flags |= XKV_FLAG_LOGITS_ONLY;
    if (!recon_tc_supported(t) || (layers[i].flags & XKV_FLAG_FORCE_GENERIC)) return false;
    const xkv_decode_params &a = layers[0], &b = layers[i];
    if (a.q_sb != b.q_sb || a.q_sh != b.q_sh || a.sm_scale != b.sm_scale || a.theta != b.theta ||
        a.pos_offset != b.pos_offset || a.inv_freq != b.inv_freq || a.k != b.k || a.k_sb != b.k_sb ||
        a.k_sl != b.k_sl || (a.kp_sb != 0) != (b.kp_sb != 0) || a.kv_lens != b.kv_lens)
      return false;
  }
  return true;
}

bool recon_tc_logits_plan(const xkv_decode_params* layers, int n, ReconTcPlan* pl) {
  xkv_decode_params t = layers[0];
  t.flags |= XKV_FLAG_LOGITS_ONLY;
  return plan_layers(t, n, pl);
}

}  // namespace xkv
