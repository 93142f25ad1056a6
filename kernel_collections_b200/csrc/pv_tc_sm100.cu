// Second pass of the two-pass decode on tcgen05: softmax over fp32 logits and P . A_v with the output
// resident in TMEM.
//
// The heads of all layers of a call are stacked on the M dimension (128 per CTA); one CTA owns up
// to 512 value columns of one (KV split, batch row): O[128 heads x 512] lives in the 512 TMEM columns
// for the whole split, the value latent streams through a TMA ring in 64-token tiles and is read from
// HBM exactly once per column block.  Eight warps:
//   warp 0      TMA producer for the value tiles (64 tokens x <=512 columns, 64-column swizzled boxes)
//   warp 1      tcgen05.mma issuer: O += P_tile . V_tile, A = P (K-major, written by the softmax
//               warps), B = the value tile (MN-major), N = 256 per instruction
//   warp 2      TMEM allocation
//   warps 4-7   softmax, ONE THREAD PER HEAD ROW (= TMEM lane): 64 logits per tile straight from
//               global memory one tile ahead, exp2 against a lazily updated reference maximum,
//               P -> shared memory as bf16, row sum in a register
// Lazy rescale: the reference maximum of a row moves only when the tile maximum exceeds it by more
// than 8 (log2 units), so P stays below 2^8 and the TMEM rows are rescaled (tcgen05.ld / st, after
// the MMAs in flight have drained) only on the rare tiles where some row moved.
// Output: normalised partials + log-sum-exp per split; the caller merges and applies B_v per layer.
#include "sm100_common.cuh"

namespace xkv {
using namespace sm100;
namespace {

constexpr int TK = 64;                      // tokens per tile
constexpr int MAXC = 512;                   // value columns per CTA (TMEM columns)
constexpr int STAGES = 3;
constexpr int STAGE_BYTES = TK * MAXC * 2;  // 64 KB
constexpr int BOX_BYTES = TK * 128;         // one 64-column box: 8 KB
constexpr int P_BYTES = 128 * TK * 2;       // 16 KB: 128 head rows x 64 tokens
constexpr int NTHREADS = 256;
constexpr int OFF_V = 0;
constexpr int OFF_P = OFF_V + STAGES * STAGE_BYTES;       // 196608
constexpr int OFF_BAR = OFF_P + 2 * P_BYTES;              // 229376
constexpr int OFF_MISC = OFF_BAR + 16 * 8;
constexpr int SMEM_BYTES = OFF_MISC + 16 + 1024;
static_assert(SMEM_BYTES <= 232448, "shared memory budget exceeded");
constexpr float RESCALE_THRESHOLD = 8.f;

struct Args {
  int batch, kv_len, heads, rv;             // stacked heads, value rank
  int num_splits, tiles_per_row, col_blocks, head_blocks;
  const float* logits;                      // [b * lg_sb + h * lg_sh + token], already times sm_scale
  int64_t lg_sb, lg_sh;
  float* partial_o;                         // [batch][heads][splits][rv]
  float* lse;                               // [batch][heads][splits]
  int* status;
  const int32_t* kv_lens;
};

template <typename T>
__global__ void __launch_bounds__(NTHREADS, 1)
pv_tc_kernel(const __grid_constant__ CUtensorMap tmV, const Args a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x;
  const int cb = blockIdx.y % a.col_blocks, hb = blockIdx.y / a.col_blocks, b = blockIdx.z;
  const int col0 = cb * MAXC;
  const int nc = min(MAXC, a.rv - col0);                 // columns of this CTA (multiple of 128)
  const int row_len = a.kv_lens ? min(max(a.kv_lens[b], 0), a.kv_len) : a.kv_len;
  const int row_tiles = a.kv_lens ? (row_len + TK - 1) / TK : a.tiles_per_row;
  const int tile_begin = (int)(((int64_t)split * row_tiles) / a.num_splits);
  const int tile_end = (int)(((int64_t)(split + 1) * row_tiles) / a.num_splits);
  const uint32_t stage_bytes = (uint32_t)(nc / 64) * BOX_BYTES;

  const uint32_t bar0 = base + OFF_BAR;
  auto bar_vfull = [&](int s) { return bar0 + 8u * s; };
  auto bar_vempty = [&](int s) { return bar0 + 8u * (4 + s); };
  auto bar_pfull = [&](int i) { return bar0 + 8u * (8 + i); };
  auto bar_pempty = [&](int i) { return bar0 + 8u * (10 + i); };
  const uint32_t bar_odone = bar0 + 8u * 12;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_MISC + 4);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(bar_vfull(s), 1); mbar_init(bar_vempty(s), 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(bar_pfull(i), 128); mbar_init(bar_pempty(i), 1); }
    mbar_init(bar_odone, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(base + OFF_MISC), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // =========================== value-tile producer ===========================================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = tile_begin; tile < tile_end; ++tile) {
        if (!mbar_wait(bar_vempty(stage), phase ^ 1u, abort_flag)) {
          report(a.status, XKV_ERR_TIMEOUT, 20, tile, cb, b);
          break;
        }
        mbar_expect_tx(bar_vfull(stage), stage_bytes);
        const uint32_t sv = base + OFF_V + stage * STAGE_BYTES;
        for (int i = 0; i < nc / 64; ++i)
          tma_load_3d(sv + i * BOX_BYTES, &tmV, col0 + i * 64, tile * TK, b, bar_vfull(stage));
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ====================================================
    if (lane == 0) {
      const int n0 = nc < 256 ? nc : 256, n1 = nc - n0;          // one or two instructions per k-step
      auto idesc_for = [&](int n) {
        return (1u << 4) | (TypeTraits<T>::kFmt << 7) | (TypeTraits<T>::kFmt << 10) | (1u << 16) |
               (((uint32_t)n >> 3) << 17) | ((128u >> 4) << 24);
      };
      const uint32_t id0 = idesc_for(n0), id1 = idesc_for(n1 > 0 ? n1 : 16);
      int stage = 0, pbuf = 0;
      uint32_t vph = 0, pph = 0;
      bool first = true;
      // operand descriptors built once; the loop only adds offsets
      const uint64_t dp0 = smem_desc(base + OFF_P, 16, 1024), dv0 = smem_desc(base + OFF_V, BOX_BYTES, 1024);
      for (int tile = tile_begin; tile < tile_end; ++tile) {
        if (!mbar_wait(bar_pfull(pbuf), pph, abort_flag) || !mbar_wait(bar_vfull(stage), vph, abort_flag)) {
          report(a.status, XKV_ERR_TIMEOUT, 21, tile, cb, b);
          goto mma_done;
        }
        tc_fence_after();
        const uint64_t da_b = desc_advance(dp0, (uint32_t)(pbuf * P_BYTES));           // P: K-major
        const uint64_t db_b = desc_advance(dv0, (uint32_t)(stage * STAGE_BYTES));      // V: MN-major
#pragma unroll
        for (int k4 = 0; k4 < TK / 16; ++k4) {
          const uint64_t da = desc_advance(da_b, k4 * 32);
          tc_mma(tmem_base, da, desc_advance(db_b, k4 * 2048), id0, (first && k4 == 0) ? 0u : 1u);
          if (n1 > 0)
            tc_mma(tmem_base + 256u, da, desc_advance(db_b, 4 * BOX_BYTES + k4 * 2048), id1, (first && k4 == 0) ? 0u : 1u);
        }
        first = false;
        tc_commit(bar_vempty(stage));       // the value tile and ...
        tc_commit(bar_pempty(pbuf));        // ... the P buffer are free once these MMAs have run
        if (++stage == STAGES) { stage = 0; vph ^= 1u; }
        pbuf ^= 1;
        if (pbuf == 0) pph ^= 1u;
      }
      tc_commit(bar_odone);
    }
  mma_done:;
  } else if (warp >= 4) {
    // =========================== softmax: one thread per head row ================================
    const int r = threadIdx.x - 128;                         // row = TMEM lane
    const int h = hb * 128 + r;
    const bool live = h < a.heads;
    const float* lrow = a.logits + (int64_t)b * a.lg_sb + (int64_t)(live ? h : 0) * a.lg_sh;
    const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const float LOG2E = 1.4426950408889634f;
    float m_ref = -CUDART_INF_F;                             // reference maximum the exponentials use
    float l_sum = 0.f;
    float cur[TK], nxt[TK];
    // a row's 64 logits of a tile: 16-byte loads when the row is aligned and the tile lies inside the row
    const bool vec_ok = (a.lg_sh % 4 == 0) && (a.lg_sb % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.logits) & 15u) == 0);
    auto fetch = [&](int tile, float (&dst)[TK]) {
      const int t0 = tile * TK;
      if (vec_ok && live && tile < tile_end && t0 + TK <= row_len) {
        const float4* src = reinterpret_cast<const float4*>(lrow + t0);
#pragma unroll
        for (int i = 0; i < TK / 4; ++i) {
          const float4 v = __ldg(src + i);
          dst[4 * i] = v.x * LOG2E; dst[4 * i + 1] = v.y * LOG2E; dst[4 * i + 2] = v.z * LOG2E; dst[4 * i + 3] = v.w * LOG2E;
        }
        return;
      }
#pragma unroll
      for (int i = 0; i < TK; ++i) {
        const int tk = t0 + i;
        dst[i] = (live && tile < tile_end && tk < row_len) ? __ldg(lrow + tk) * LOG2E : -CUDART_INF_F;
      }
    };
    // The register loads run one tile ahead, which covers an L2 hit but not a trip to HBM: the row's 256 bytes of
    // the tile three ahead are asked into L2 meanwhile (two 128-byte lines; a hint, so a line past the row is harmless
    // as long as it lies inside the logits buffer, which the tile_end test guarantees).
    auto prefetch_l2 = [&](int tile) {
      if (live && tile < tile_end && (tile + 1) * TK <= row_len) {
        const float* pf = lrow + (int64_t)tile * TK;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(pf));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(pf + 32));
      }
    };
    prefetch_l2(tile_begin + 1);
    prefetch_l2(tile_begin + 2);
    fetch(tile_begin, nxt);
    int pbuf = 0;
    uint32_t pph = 0;
    for (int tile = tile_begin; tile < tile_end; ++tile) {
#pragma unroll
      for (int i = 0; i < TK; ++i) cur[i] = nxt[i];
      prefetch_l2(tile + 3);
      fetch(tile + 1, nxt);
      float tmax = -CUDART_INF_F;
#pragma unroll
      for (int i = 0; i < TK; ++i) tmax = fmaxf(tmax, cur[i]);
      // does this row's reference have to move?  (first finite tile, or the tile tops it by > 8)
      const bool move = tmax > m_ref + RESCALE_THRESHOLD || (m_ref == -CUDART_INF_F && tmax > -CUDART_INF_F);
      // all 128 rows agree on whether to rescale (barrier with reduction), so the TMEM pass is uniform
      // (one barrier per tile: a raised abort flag rides on the same vote and is told apart by a second, rare one)
      auto vote = [](uint32_t mine) -> uint32_t {
        uint32_t res;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.u32 p, %1, 0;\n\t"
            "barrier.cta.red.or.pred q, 1, 128, p;\n\t"
            "selp.u32 %0, 1, 0, q;\n\t}"
            : "=r"(res)
            : "r"(mine)
            : "memory");
        return res;
      };
      const uint32_t any = vote((move || *abort_flag) ? 1u : 0u);
      if (any && vote(*abort_flag ? 1u : 0u)) break;
      if (any) {
        const float m_new = move ? tmax : m_ref;
        const float alpha = (m_ref == -CUDART_INF_F) ? 0.f : exp2f(m_ref - m_new);
        if (tile > tile_begin) {
          // wait until the MMAs issued so far have drained (the previous tile's P buffer is released by
          // the commit that follows them), then rescale this row of O in place
          if (!mbar_wait(bar_pempty(pbuf ^ 1), pbuf == 1 ? pph : pph ^ 1u, abort_flag))
            report(a.status, XKV_ERR_TIMEOUT, 23, tile, cb, b);
          tc_fence_after();
          for (int c = 0; c < nc; c += 32) {
            uint32_t v[32];
            tmem_ld32(lane_addr + c, v);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st32(lane_addr + c, v);
          }
          tmem_wait_st();
          tc_fence_before();
        }
        l_sum *= alpha;
        m_ref = m_new;
      }
      if (a.kv_lens != nullptr && (tile + 1) * TK > row_len) {
        // Ragged batch, last tile of the row: value rows past the row's own length are outside the
        // call (they may hold anything, NaN included, and 0 * NaN is NaN).  Once the tile has landed
        // the softmax threads zero those rows; the proxy fence before the P hand-over below orders
        // the stores ahead of the MMAs that read the tile.
        const int it = tile - tile_begin, vstage = it % STAGES;
        if (!mbar_wait(bar_vfull(vstage), (uint32_t)(it / STAGES) & 1u, abort_flag))
          report(a.status, XKV_ERR_TIMEOUT, 26, tile, cb, b);
        const int first = max(row_len - tile * TK, 0), per_row = (nc / 64) * 8;
        for (int idx = r; idx < (TK - first) * per_row; idx += 128) {
          const int row = first + idx / per_row, rem = idx % per_row;
          *reinterpret_cast<uint4*>(sm + OFF_V + vstage * STAGE_BYTES + (rem >> 3) * BOX_BYTES + row * 128 + (rem & 7) * 16) =
              make_uint4(0u, 0u, 0u, 0u);
        }
      }
      // ---- P row -> shared memory (K-major, 128-byte swizzle), row sum of the rounded values ----------
      if (!mbar_wait(bar_pempty(pbuf), pph ^ 1u, abort_flag)) report(a.status, XKV_ERR_TIMEOUT, 24, tile, cb, b);
      const float mref = m_ref == -CUDART_INF_F ? 0.f : m_ref;
      uint8_t* prow = sm + OFF_P + pbuf * P_BYTES + r * 128;
#pragma unroll
      for (int c8 = 0; c8 < TK / 8; ++c8) {
        uint32_t pk[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          pk[i] = TypeTraits<T>::pack2(exp2f(cur[c8 * 8 + 2 * i] - mref), exp2f(cur[c8 * 8 + 2 * i + 1] - mref));
          const float2 q = TypeTraits<T>::unpack2(pk[i]);
          l_sum += q.x + q.y;
        }
        *reinterpret_cast<uint4*>(prow + ((c8 ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> tcgen05 (async proxy) reads
      mbar_arrive(bar_pfull(pbuf));
      pbuf ^= 1;
      if (pbuf == 0) pph ^= 1u;
    }
    // ---- output: O row / l, log-sum-exp ------------------------------------------------------------------
    if (!*abort_flag && tile_end > tile_begin) {
      if (!mbar_wait(bar_odone, 0, abort_flag)) report(a.status, XKV_ERR_TIMEOUT, 25, tile_end, cb, b);
      tc_fence_after();
    }
    if (!*abort_flag) {
      const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
      float* po = a.partial_o + (((int64_t)b * a.heads + (live ? h : 0)) * a.num_splits + split) * a.rv + col0;
      for (int c = 0; c < nc; c += 32) {
        uint32_t v[32];
        if (tile_end > tile_begin) {          // (warp-wide TMEM load: rows past the last head take part)
          tmem_ld32(lane_addr + c, v);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (live) {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(po + c + i) =
                make_float4(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv,
                            __uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
        }
      }
      if (live && cb == 0)
        a.lse[((int64_t)b * a.heads + h) * a.num_splits + split] =
            l_sum > 0.f ? (m_ref + log2f(l_sum)) * 0.6931471805599453f : -CUDART_INF_F;
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

template <typename T>
int launch(const CUtensorMap& tV, const Args& a, cudaStream_t st) {
  auto kern = pv_tc_kernel<T>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) {
    cudaGetLastError();
    return XKV_ERR_LAUNCH;
  }
  kern<<<dim3(a.num_splits, a.col_blocks * a.head_blocks, a.batch), NTHREADS, SMEM_BYTES, st>>>(tV, a);
  return cudaGetLastError() == cudaSuccess ? XKV_OK : XKV_ERR_LAUNCH;
}

}  // namespace

bool pv_tc_supported(const xkv_decode_params& p) {
  if (p.value_mode != XKV_VALUE_LATENT || (p.flags & (XKV_FLAG_LOGITS_ONLY | XKV_FLAG_FORCE_GENERIC))) return false;
  if (p.dtype != XKV_BF16 && p.dtype != XKV_F16) return false;
  if (p.v_rank % 128 != 0 || p.v_rank > 4096 || p.logit_cap > 0.f || p.tail_dim != 0 || p.mask) return false;
  if (!aligned16(p.v) || !stride_ok(p.v_sl) || (p.batch > 1 && !stride_ok(p.v_sb))) return false;
  return true;
}

bool pv_tc_plan(const xkv_decode_params& p, int heads, PvTcPlan* pl) {
  pl->col_blocks = ceil_div(p.v_rank, MAXC);
  pl->head_blocks = ceil_div(heads, 128);
  pl->tiles = ceil_div(p.kv_len, TK);
  const int rows = p.batch * pl->col_blocks * pl->head_blocks;
  const int sms = device_sm_count();
  int best_s = 1;
  int64_t best_cost = -1;
  const int max_s = pl->tiles < 64 ? pl->tiles : 64;
  for (int s = 1; s <= max_s; ++s) {
    const int64_t waves = ceil_div(rows * s, sms);
    const int64_t cost = waves * (ceil_div(pl->tiles, s) + 4);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_s = s; }
  }
  pl->num_splits = best_s;
  size_t off = 0;
  pl->off_partial = off;
  off += align_up((size_t)p.batch * heads * best_s * p.v_rank * sizeof(float), 256);
  pl->off_lse = off;
  off += align_up((size_t)p.batch * heads * best_s * sizeof(float), 256);
  pl->total_bytes = off;
  return true;
}

int pv_tc_run(const xkv_decode_params& p, int heads, const PvTcPlan& pl, const float* logits, void* ws, int* status,
              cudaStream_t st) {
  char* w = static_cast<char*>(ws);
  CUtensorMap tV;
  {
    const cuuint64_t dims[3] = {(cuuint64_t)p.v_rank, (cuuint64_t)p.kv_len, (cuuint64_t)p.batch};
    const int64_t sb = p.batch > 1 ? p.v_sb : (int64_t)p.kv_len * p.v_sl;
    const cuuint64_t strides[2] = {(cuuint64_t)p.v_sl * 2, (cuuint64_t)sb * 2};
    const cuuint32_t box[3] = {64, TK, 1};
    if (!encode_tiled_16bit(&tV, p.dtype, 3, p.v, dims, strides, box)) return XKV_ERR_NO_DEVICE;
  }
  Args a;
  a.batch = p.batch; a.kv_len = p.kv_len; a.heads = heads; a.rv = p.v_rank;
  a.num_splits = pl.num_splits; a.tiles_per_row = pl.tiles; a.col_blocks = pl.col_blocks; a.head_blocks = pl.head_blocks;
  a.logits = logits; a.lg_sb = (int64_t)heads * p.kv_len; a.lg_sh = p.kv_len;
  a.partial_o = reinterpret_cast<float*>(w + pl.off_partial);
  a.lse = reinterpret_cast<float*>(w + pl.off_lse);
  a.status = status;
  a.kv_lens = p.kv_lens;
  return p.dtype == XKV_BF16 ? launch<__nv_bfloat16>(tV, a, st) : launch<__half>(tV, a, st);
}

}  // namespace xkv
