// Portable CUDA-core decode-attention path: every score / value mode, every dtype, any shape
// within the size limits.  It is the path fp32 inputs and odd shapes take; the tensor-core
// kernels take over for the aligned bf16 / fp16 shapes they cover.
//
// Three launches per call:
//   1. absorb_query_kernel   q_eff[b,h,:] = q . k_proj^T (latent scores) or a plain fp32 copy,
//                            with the decoupled RoPE query part appended.
//   2. decode_partial_kernel split-KV pass: per (split, batch row, head chunk) builds 16-token
//                            key tiles in shared memory (dense rows, latent rows, or rows
//                            rebuilt as A.B and rotated), scores them against the chunk's
//                            query heads, runs an online softmax and accumulates P.V.
//   3. merge_kernel          log-sum-exp weighted merge of the splits, in split order (results
//                            are run-to-run identical), then the optional value projection.
#include "xkv_internal.h"
#include <math_constants.h>
#include <mutex>

namespace xkv {
namespace {

constexpr int TT = 16;             // tokens per tile
constexpr int NT = 256;            // threads per CTA of the split-KV pass
constexpr int HC_MAX = 16;         // query heads per CTA
constexpr int ACC_PER_THREAD = 4;  // accumulated value columns per thread -> acc_dim <= 1024
constexpr int RECON_PER_THREAD = 16;  // rebuilt key elements per thread -> head_dim <= 256
constexpr int MAX_SPLITS = 512;

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <> __device__ __forceinline__ float ldf<__half>(const __half* p) { return __half2float(*p); }

template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ void stf<__half>(__half* p, float v) { *p = __float2half_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void absorb_query_kernel(const xkv_decode_params p, float* __restrict__ qeff,
                                    int score_dim, int* __restrict__ status) {
  extern __shared__ float q_s[];
  const int h = blockIdx.x, b = blockIdx.y;
  if (h == 0 && b == 0 && threadIdx.x < 8) status[threadIdx.x] = 0;  // this path never waits: always "ok"
  const T* q = static_cast<const T*>(p.q) + (int64_t)b * p.q_sb + (int64_t)h * p.q_sh;
  float* out = qeff + ((int64_t)b * p.num_heads + h) * score_dim;
  for (int d = threadIdx.x; d < p.head_dim; d += blockDim.x) q_s[d] = ldf(q + d);
  __syncthreads();
  int main_dim;
  if (p.score_mode == XKV_SCORE_LATENT && p.k_proj != nullptr) {
    main_dim = p.k_rank;
    const int div = p.num_heads / p.k_proj_heads;
    const T* kp = static_cast<const T*>(p.k_proj) + (int64_t)b * p.kp_sb + (int64_t)(h / div) * p.kp_sh;
    for (int r = threadIdx.x; r < p.k_rank; r += blockDim.x) {
      const T* row = kp + (int64_t)r * p.kp_sr;
      float acc = 0.f;
      for (int d = 0; d < p.head_dim; ++d) acc = fmaf(q_s[d], ldf(row + (int64_t)d * p.kp_sd), acc);
      out[r] = acc;
    }
  } else {
    main_dim = p.head_dim;
    for (int d = threadIdx.x; d < p.head_dim; d += blockDim.x) out[d] = q_s[d];
  }
  if (p.tail_dim > 0) {
    const T* qt = static_cast<const T*>(p.q_tail) + (int64_t)b * p.qt_sb + (int64_t)h * p.qt_sh;
    for (int d = threadIdx.x; d < p.tail_dim; d += blockDim.x) out[main_dim + d] = ldf(qt + d);
  }
}

// ---------------------------------------------------------------------------------------------
struct PartialGeom {
  int heads_per_cta, num_splits, split_len, score_dim, acc_dim;
};

template <typename T>
__global__ void __launch_bounds__(NT)
decode_partial_kernel(const xkv_decode_params p, const PartialGeom g, const float* __restrict__ qeff,
                      float* __restrict__ partial_o, float* __restrict__ lse_out) {
  extern __shared__ float smem[];
  const int HC = g.heads_per_cta, Dq = g.score_dim, Dacc = g.acc_dim;
  float* q_s = smem;                       // [HC][Dq]
  float* k_s = q_s + HC * Dq;              // [TT][Dq]
  float* logit_s = k_s + TT * Dq;          // [HC_MAX][TT]
  float* prob_s = logit_s + HC_MAX * TT;   // [HC_MAX][TT]
  float* alpha_s = prob_s + HC_MAX * TT;   // [HC_MAX]
  float* m_s = alpha_s + HC_MAX;           // [HC_MAX]
  float* l_s = m_s + HC_MAX;               // [HC_MAX]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x, b = blockIdx.y, h0 = blockIdx.z * HC;
  const int H = p.num_heads;
  const int L = p.kv_lens ? min(max(p.kv_lens[b], 0), p.kv_len) : p.kv_len;   // this row's length
  const int G = H / p.num_kv_heads;
  const int kvh = h0 / G;
  const int tok_begin = split * g.split_len;
  const int tok_end = min(L, tok_begin + g.split_len);
  const bool logits_only = (p.flags & XKV_FLAG_LOGITS_ONLY) != 0;

  for (int i = tid; i < HC * Dq; i += NT) q_s[i] = qeff[((int64_t)b * H + h0) * Dq + i];
  if (tid < HC_MAX) { m_s[tid] = -CUDART_INF_F; l_s[tid] = 0.f; }

  float acc[HC_MAX][ACC_PER_THREAD];
#pragma unroll
  for (int h = 0; h < HC_MAX; ++h)
#pragma unroll
    for (int i = 0; i < ACC_PER_THREAD; ++i) acc[h][i] = 0.f;

  const T* kbase = static_cast<const T*>(p.k) + (int64_t)b * p.k_sb;
  const T* ktail = p.k_tail ? static_cast<const T*>(p.k_tail) + (int64_t)b * p.kt_sb : nullptr;
  const T* vbase = static_cast<const T*>(p.v);
  if (vbase) vbase += (int64_t)b * p.v_sb + (p.value_mode == XKV_VALUE_DENSE ? (int64_t)kvh * p.v_sh : 0);
  const int D = p.head_dim;
  __syncthreads();

  for (int base = tok_begin; base < tok_end; base += TT) {
    // ---- phase A: key tile -> k_s (fp32) -------------------------------------------------
    if (p.score_mode == XKV_SCORE_DENSE) {
      const T* kk = kbase + (int64_t)kvh * p.k_sh;
      for (int idx = tid; idx < TT * D; idx += NT) {
        const int t = idx / D, d = idx - t * D, tok = base + t;
        k_s[t * Dq + d] = tok < tok_end ? ldf(kk + (int64_t)tok * p.k_sl + d) : 0.f;
      }
    } else if (p.score_mode == XKV_SCORE_LATENT) {
      const int R = p.k_rank;
      for (int idx = tid; idx < TT * Dq; idx += NT) {
        const int t = idx / Dq, d = idx - t * Dq, tok = base + t;
        float v = 0.f;
        if (tok < tok_end)
          v = d < R ? ldf(kbase + (int64_t)tok * p.k_sl + d) : ldf(ktail + (int64_t)tok * p.kt_sl + (d - R));
        k_s[idx] = v;
      }
    } else {
      // rebuild K[t, d] = sum_r A[t, r] * B[kvh, r, d]
      const T* bp = static_cast<const T*>(p.k_proj) + (int64_t)b * p.kp_sb + (int64_t)kvh * p.kp_sh;
      float kacc[RECON_PER_THREAD];
      int tt[RECON_PER_THREAD], dd[RECON_PER_THREAD];
#pragma unroll
      for (int i = 0; i < RECON_PER_THREAD; ++i) {
        const int idx = tid + i * NT;
        kacc[i] = 0.f;
        tt[i] = idx / D;
        dd[i] = idx - tt[i] * D;
      }
      for (int r = 0; r < p.k_rank; ++r) {
        const T* brow = bp + (int64_t)r * p.kp_sr;
#pragma unroll
        for (int i = 0; i < RECON_PER_THREAD; ++i) {
          const int tok = base + tt[i];
          if (tid + i * NT < TT * D && tok < tok_end)
            kacc[i] = fmaf(ldf(kbase + (int64_t)tok * p.k_sl + r), ldf(brow + (int64_t)dd[i] * p.kp_sd), kacc[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < RECON_PER_THREAD; ++i)
        if (tid + i * NT < TT * D) k_s[tt[i] * Dq + dd[i]] = kacc[i];
      if (p.score_mode == XKV_SCORE_RECON_ROPE) {
        __syncthreads();
        const int half = D / 2;
        for (int idx = tid; idx < TT * half; idx += NT) {
          const int t = idx / half, j = idx - t * half;
          float sn, cs;
          if (p.rope_table) {
            const int row = min(base + t, L - 1);
            const float2 t2 = reinterpret_cast<const float2*>(p.rope_table)[(int64_t)row * half + j];
            cs = t2.x;
            sn = t2.y;
          } else {
            const float f = p.inv_freq ? p.inv_freq[j] : 1.0f / powf(p.theta, (float)(2 * j) / (float)D);
            sincosf(__fmul_rn((float)(p.pos_offset + base + t), f), &sn, &cs);
          }
          const float x0 = k_s[t * Dq + j], x1 = k_s[t * Dq + j + half];
          k_s[t * Dq + j] = x0 * cs - x1 * sn;
          k_s[t * Dq + j + half] = x1 * cs + x0 * sn;
        }
      }
    }
    __syncthreads();

    // ---- phase B: logits = q_eff . key rows ------------------------------------------------
    for (int t = warp; t < TT; t += NT / 32) {
      const int tok = base + t;
      float part[HC_MAX];
#pragma unroll
      for (int h = 0; h < HC_MAX; ++h) part[h] = 0.f;
      for (int d = lane; d < Dq; d += 32) {
        const float kv = k_s[t * Dq + d];
#pragma unroll
        for (int h = 0; h < HC_MAX; ++h)
          if (h < HC) part[h] = fmaf(q_s[h * Dq + d], kv, part[h]);
      }
#pragma unroll
      for (int h = 0; h < HC_MAX; ++h) {
        if (h < HC) {
          float s = warp_sum(part[h]) * p.sm_scale;
          if (p.logit_cap > 0.f) s = p.logit_cap * tanhf(s / p.logit_cap);
          if (p.mask && tok < tok_end)
            s += ldf(static_cast<const T*>(p.mask) + (int64_t)b * p.mask_sb + (int64_t)(h0 + h) * p.mask_sh + tok);
          if (lane == 0) {
            if (logits_only) {
              if (tok < tok_end)
                stf(static_cast<T*>(p.logits) + (int64_t)b * p.lg_sb + (int64_t)(h0 + h) * p.lg_sh + tok, s);
            } else {
              logit_s[h * TT + t] = tok < tok_end ? s : -CUDART_INF_F;
            }
          }
        }
      }
    }
    __syncthreads();
    if (logits_only) continue;

    // ---- phase C: online softmax, one thread per head --------------------------------------
    if (tid < HC) {
      const int h = tid;
      float mx = m_s[h];
#pragma unroll
      for (int t = 0; t < TT; ++t) mx = fmaxf(mx, logit_s[h * TT + t]);
      // a tile masked to -inf before anything finite was seen leaves the maximum at -inf: keep the
      // exponentials finite (they are all zero) instead of forming exp(-inf - -inf)
      const float m_use = (mx == -CUDART_INF_F) ? 0.f : mx;
      const float alpha = (m_s[h] == -CUDART_INF_F) ? 0.f : expf(m_s[h] - m_use);
      float sum = 0.f;
#pragma unroll
      for (int t = 0; t < TT; ++t) {
        const float e = expf(logit_s[h * TT + t] - m_use);
        prob_s[h * TT + t] = e;
        sum += e;
      }
      alpha_s[h] = alpha;
      l_s[h] = l_s[h] * alpha + sum;
      m_s[h] = mx;
    }
    __syncthreads();

    // ---- phase D: acc = acc * alpha + P . V ------------------------------------------------
#pragma unroll
    for (int h = 0; h < HC_MAX; ++h)
      if (h < HC) {
        const float a = alpha_s[h];
#pragma unroll
        for (int i = 0; i < ACC_PER_THREAD; ++i) acc[h][i] *= a;
      }
    const int ntok = min(TT, tok_end - base);
    for (int t = 0; t < ntok; ++t) {
      const T* vrow = vbase + (int64_t)(base + t) * p.v_sl;
      float vv[ACC_PER_THREAD];
#pragma unroll
      for (int i = 0; i < ACC_PER_THREAD; ++i) {
        const int c = tid + i * NT;
        vv[i] = c < Dacc ? ldf(vrow + c) : 0.f;
      }
#pragma unroll
      for (int h = 0; h < HC_MAX; ++h)
        if (h < HC) {
          const float pr = prob_s[h * TT + t];
#pragma unroll
          for (int i = 0; i < ACC_PER_THREAD; ++i) acc[h][i] = fmaf(pr, vv[i], acc[h][i]);
        }
    }
    __syncthreads();
  }
  if (logits_only) return;

  // ---- finalize: normalised partial + log-sum-exp -------------------------------------------
#pragma unroll
  for (int h = 0; h < HC_MAX; ++h)
    if (h < HC) {
      const float l = l_s[h];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      float* po = partial_o + (((int64_t)b * H + h0 + h) * g.num_splits + split) * Dacc;
#pragma unroll
      for (int i = 0; i < ACC_PER_THREAD; ++i) {
        const int c = tid + i * NT;
        if (c < Dacc) po[c] = acc[h][i] * inv;
      }
    }
  if (tid < HC) {
    const float l = l_s[tid];
    lse_out[((int64_t)b * H + h0 + tid) * g.num_splits + split] = l > 0.f ? m_s[tid] + logf(l) : -CUDART_INF_F;
  }
}

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(NT)
merge_kernel(const float* __restrict__ partial_o, const float* __restrict__ lse, T* __restrict__ out,
             int num_heads, int heads_total, int head_offset, int S, int Dacc, int Dv, const T* __restrict__ v_proj, int v_div,
             int64_t vp_sb, int64_t vp_sh, int64_t vp_sr, int64_t vp_sd, int64_t o_sb, int64_t o_sh,
             int vec_proj, float* __restrict__ lse_out, int64_t lse_sb) {
  extern __shared__ float smem[];
  float* w_s = smem;          // [S]
  float* o_s = smem + S;      // [Dacc]
  __shared__ float red[NT / 32];
  __shared__ float bcast[2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.x, b = blockIdx.y;
  // the partials may belong to a wider buffer of stacked heads (several layers side by side)
  const int64_t prow = (int64_t)b * heads_total + head_offset + h;
  const float* ls = lse + prow * S;
  const float* po = partial_o + prow * S * (int64_t)Dacc;
  (void)num_heads;

  float mx = -CUDART_INF_F;
  for (int s = tid; s < S; s += NT) mx = fmaxf(mx, ls[s]);
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  if (tid == 0) {
    float m = red[0];
    for (int i = 1; i < NT / 32; ++i) m = fmaxf(m, red[i]);
    bcast[0] = m;
  }
  __syncthreads();
  mx = bcast[0];
  for (int s = tid; s < S; s += NT) {
    const float v = ls[s];
    w_s[s] = (v == -CUDART_INF_F) ? 0.f : expf(v - mx);
  }
  __syncthreads();
  if (tid == 0) {
    float tot = 0.f;
    for (int s = 0; s < S; ++s) tot += w_s[s];  // fixed order
    bcast[1] = tot > 0.f ? 1.f / tot : 0.f;
    // log-sum-exp over the whole row, for callers that merge several calls
    if (lse_out) lse_out[(int64_t)b * lse_sb + h] = tot > 0.f ? mx + logf(tot) : -CUDART_INF_F;
  }
  __syncthreads();
  const float inv = bcast[1];
  for (int c = tid; c < Dacc; c += NT) {
    float o = 0.f;
    for (int s = 0; s < S; ++s) {
      const float w = w_s[s];
      if (w != 0.f) o = fmaf(w, po[(int64_t)s * Dacc + c], o);
    }
    o_s[c] = o * inv;
  }
  __syncthreads();
  T* orow = out + (int64_t)b * o_sb + (int64_t)h * o_sh;
  if (v_proj == nullptr) {
    for (int c = tid; c < Dacc; c += NT) stf(orow + c, o_s[c]);
  } else if (vec_proj) {
    // out[d] = sum_r o[r] * v_proj[r, d] with 16-byte loads: the threads form Dv / VEC column lanes
    // times NT / lanes row groups; each group walks its share of the rank, the groups are then added
    // in a fixed order.
    constexpr int VEC = 16 / (int)sizeof(T);
    __shared__ float part_s[NT * VEC];
    const int lanes = Dv / VEC, groups = NT / lanes;
    const int ln = tid % lanes, grp = tid / lanes;
    float part[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) part[e] = 0.f;
    const T* vp = v_proj + (int64_t)b * vp_sb + (int64_t)(h / v_div) * vp_sh + ln * VEC;
    if (grp < groups) {
      for (int r = grp; r < Dacc; r += groups) {
        const uint4 raw = *reinterpret_cast<const uint4*>(vp + (int64_t)r * vp_sr);
        const T* e8 = reinterpret_cast<const T*>(&raw);
        const float o = o_s[r];
#pragma unroll
        for (int e = 0; e < VEC; ++e) part[e] = fmaf(o, ldf(e8 + e), part[e]);
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) part_s[grp * Dv + ln * VEC + e] = part[e];
    }
    __syncthreads();
    for (int d = tid; d < Dv; d += NT) {
      float o = 0.f;
      for (int k = 0; k < groups; ++k) o += part_s[k * Dv + d];
      stf(orow + d, o);
    }
  } else {
    const T* vp = v_proj + (int64_t)b * vp_sb + (int64_t)(h / v_div) * vp_sh;
    for (int d = tid; d < Dv; d += NT) {
      float o = 0.f;
      for (int r = 0; r < Dacc; ++r) o = fmaf(o_s[r], ldf(vp + (int64_t)r * vp_sr + (int64_t)d * vp_sd), o);
      stf(orow + d, o);
    }
  }
}

__global__ void rope_table_kernel(float2* __restrict__ cos_sin, int kv_len, int half, int pos_offset,
                                  float theta, const float* __restrict__ inv_freq) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)kv_len * half) return;
  const int l = (int)(idx / half), j = (int)(idx - (int64_t)l * half);
  const float f = inv_freq ? inv_freq[j] : 1.0f / powf(theta, (float)(2 * j) / (float)(2 * half));
  float sn, cs;
  sincosf(__fmul_rn((float)(pos_offset + l), f), &sn, &cs);
  cos_sin[idx] = make_float2(cs, sn);
}

template <typename T>
int run_generic(const xkv_decode_params& p, const GenericPlan& pl, void* ws, cudaStream_t st) {
  char* w = static_cast<char*>(ws);
  float* qeff = reinterpret_cast<float*>(w + pl.off_qeff);
  float* partial = reinterpret_cast<float*>(w + pl.off_partial);
  float* lse = reinterpret_cast<float*>(w + pl.off_lse);
  absorb_query_kernel<T><<<dim3(p.num_heads, p.batch), 128, p.head_dim * sizeof(float), st>>>(
      p, qeff, pl.score_dim, reinterpret_cast<int*>(w));
  PartialGeom g{pl.heads_per_cta, pl.num_splits, pl.split_len, pl.score_dim, pl.acc_dim};
  // opt in to the large dynamic shared-memory carve-out (per device, cheap, idempotent)
  if (cudaFuncSetAttribute(decode_partial_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           200 * 1024) != cudaSuccess) {
    cudaGetLastError();
    return XKV_ERR_LAUNCH;
  }
  decode_partial_kernel<T><<<dim3(pl.num_splits, p.batch, pl.head_chunks), NT, pl.smem_bytes, st>>>(
      p, g, qeff, partial, lse);
  if (!(p.flags & XKV_FLAG_LOGITS_ONLY)) {
    int rc = launch_merge(partial, lse, p.out, p.dtype, p.batch, p.num_heads, pl.num_splits, pl.acc_dim,
                          p.value_dim, p.value_mode == XKV_VALUE_LATENT ? p.v_proj : nullptr,
                          p.v_proj_heads, p.vp_sb, p.vp_sh, p.vp_sr, p.vp_sd, p.o_sb, p.o_sh, st, 0, 0, p.lse_out, p.lse_sb);
    if (rc != XKV_OK) return rc;
  }
  return cudaGetLastError() == cudaSuccess ? XKV_OK : XKV_ERR_LAUNCH;
}

}  // namespace

int device_sm_count() {
  // SM count of the current device, looked up once per device
  constexpr int kMaxDevices = 64;
  static int cached[kMaxDevices] = {};
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return kNumSMsFallback;
  }
  if (dev >= 0 && dev < kMaxDevices && cached[dev] > 0) return cached[dev];
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    return kNumSMsFallback;
  }
  if (dev >= 0 && dev < kMaxDevices) cached[dev] = n;
  return n;
}

bool generic_plan(const xkv_decode_params& p, GenericPlan* pl) {
  const int G = p.num_heads / p.num_kv_heads;
  int hc = 1;
  for (int c = 1; c <= HC_MAX; ++c)
    if (G % c == 0) hc = c;
  pl->heads_per_cta = hc;
  pl->head_chunks = p.num_heads / hc;
  pl->score_dim = (p.score_mode == XKV_SCORE_LATENT ? p.k_rank : p.head_dim) + p.tail_dim;
  pl->acc_dim = p.value_mode == XKV_VALUE_LATENT ? p.v_rank : p.value_dim;
  const bool logits_only = (p.flags & XKV_FLAG_LOGITS_ONLY) != 0;
  if (logits_only) pl->acc_dim = 1;
  if (pl->acc_dim > ACC_PER_THREAD * NT) return false;
  if ((p.score_mode == XKV_SCORE_RECON || p.score_mode == XKV_SCORE_RECON_ROPE) &&
      TT * p.head_dim > RECON_PER_THREAD * NT)
    return false;
  pl->smem_bytes = ((size_t)(hc + TT) * pl->score_dim + 2 * HC_MAX * TT + 3 * HC_MAX) * sizeof(float);
  if (pl->smem_bytes > 200 * 1024) return false;
  const int tiles = ceil_div(p.kv_len, TT);
  int S;
  if (p.num_splits > 0) {
    S = p.num_splits;
  } else {
    const int target = 4 * device_sm_count();
    S = ceil_div(target, p.batch * pl->head_chunks);
  }
  if (S > tiles) S = tiles;
  if (S > MAX_SPLITS) S = MAX_SPLITS;
  if (S < 1) S = 1;
  pl->split_len = ceil_div(tiles, S) * TT;
  pl->num_splits = ceil_div(p.kv_len, pl->split_len);
  size_t off = 256;  // status words lead every workspace
  pl->off_qeff = off;
  off += align_up((size_t)p.batch * p.num_heads * pl->score_dim * sizeof(float), 256);
  pl->off_partial = off;
  if (!logits_only) off += align_up((size_t)p.batch * p.num_heads * pl->num_splits * pl->acc_dim * sizeof(float), 256);
  pl->off_lse = off;
  if (!logits_only) off += align_up((size_t)p.batch * p.num_heads * pl->num_splits * sizeof(float), 256);
  pl->total_bytes = off;
  return true;
}

int generic_decode(const xkv_decode_params& p, const GenericPlan& pl, void* ws, cudaStream_t st) {
  switch (p.dtype) {
    case XKV_F32: return run_generic<float>(p, pl, ws, st);
    case XKV_BF16: return run_generic<__nv_bfloat16>(p, pl, ws, st);
    case XKV_F16: return run_generic<__half>(p, pl, ws, st);
    default: return XKV_ERR_BAD_ARG;
  }
}

// ---- built-in scratch for callers that cannot allocate device memory ---------------------------
// One fixed array per device that loads the library, resident until the process exits.  In host
// code the symbol below is only a handle; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_builtin_scratch[XKV_BUILTIN_SCRATCH_BYTES];

int generic_decode_builtin_scratch(const xkv_decode_params& p, const GenericPlan& pl, cudaStream_t st) {
  if (pl.total_bytes > (size_t)XKV_BUILTIN_SCRATCH_BYTES) return XKV_ERR_SCRATCH_LIMIT;
  constexpr int kMaxDevices = 64;
  static void* dev_ptr[kMaxDevices] = {};
  static std::mutex mu;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return XKV_ERR_NO_DEVICE;
  }
  void* ptr = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!dev_ptr[dev]) {
      // first call on this device: resolve the array's device address (no allocation happens)
      void* sym = nullptr;
      if (cudaGetSymbolAddress(&sym, g_builtin_scratch) != cudaSuccess || !sym) {
        cudaGetLastError();
        return XKV_ERR_NO_DEVICE;
      }
      dev_ptr[dev] = sym;
    }
    ptr = dev_ptr[dev];
  }
  // Every region of the scratch that a kernel reads is written earlier in the same call: the
  // status words and q_eff by the first kernel, each (batch, head, split) partial and its
  // log-sum-exp by the split-KV pass.  Nothing relies on the previous call's contents.
  return generic_decode(p, pl, ptr, st);
}

// The same merge without a value projection, one WARP per (batch, head) row and no block-wide barriers: every
// lane walks the splits in order (same weights, same order of additions as merge_kernel, so the two agree bit for
// bit) over its own 4-column groups, with 16-byte loads of the partial rows.
template <typename T>
__global__ void __launch_bounds__(256)
merge_rows_kernel(const float* __restrict__ partial_o, const float* __restrict__ lse, T* __restrict__ out, int rows,
                  int num_heads, int heads_total, int head_offset, int S, int Dacc, int64_t o_sb, int64_t o_sh,
                  float* __restrict__ lse_out, int64_t lse_sb) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int b = row / num_heads, h = row - b * num_heads;
  const int64_t prow = (int64_t)b * heads_total + head_offset + h;
  const float* ls = lse + prow * S;
  const float* po = partial_o + prow * S * (int64_t)Dacc;
  float mx = -CUDART_INF_F;
  for (int s = 0; s < S; ++s) mx = fmaxf(mx, ls[s]);
  float tot = 0.f;
  for (int s = 0; s < S; ++s) {
    const float v = ls[s];
    tot += (v == -CUDART_INF_F) ? 0.f : expf(v - mx);
  }
  const float inv = tot > 0.f ? 1.f / tot : 0.f;
  if (lane == 0 && lse_out) lse_out[(int64_t)b * lse_sb + h] = tot > 0.f ? mx + logf(tot) : -CUDART_INF_F;
  T* orow = out + (int64_t)b * o_sb + (int64_t)h * o_sh;
  for (int c = lane * 4; c < Dacc; c += 128) {
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < S; ++s) {
      const float v = ls[s];
      const float w = (v == -CUDART_INF_F) ? 0.f : expf(v - mx);
      if (w != 0.f) {
        const float4 p4 = *reinterpret_cast<const float4*>(po + (int64_t)s * Dacc + c);
        o.x = fmaf(w, p4.x, o.x); o.y = fmaf(w, p4.y, o.y); o.z = fmaf(w, p4.z, o.z); o.w = fmaf(w, p4.w, o.w);
      }
    }
    stf(orow + c, o.x * inv); stf(orow + c + 1, o.y * inv); stf(orow + c + 2, o.z * inv); stf(orow + c + 3, o.w * inv);
  }
}

int launch_merge(const float* partial_o, const float* lse, void* out, int dtype, int batch, int num_heads,
                 int num_splits, int acc_dim, int value_dim, const void* v_proj, int v_proj_heads,
                 int64_t vp_sb, int64_t vp_sh, int64_t vp_sr, int64_t vp_sd, int64_t o_sb, int64_t o_sh,
                 cudaStream_t st, int heads_total, int head_offset, float* lse_out, int64_t lse_sb) {
  if (heads_total <= 0) heads_total = num_heads;
  if (v_proj == nullptr && value_dim == acc_dim && acc_dim % 4 == 0 && (reinterpret_cast<uintptr_t>(partial_o) & 15u) == 0) {
    const int rows = batch * num_heads;
#define XKV_MERGE_ROWS(T)                                                                                         \
  merge_rows_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(partial_o, lse, static_cast<T*>(out), rows, num_heads, \
                                                                    heads_total, head_offset, num_splits, acc_dim, o_sb, o_sh, \
                                                                    lse_out, lse_sb)
    switch (dtype) {
      case XKV_F32: XKV_MERGE_ROWS(float); break;
      case XKV_BF16: XKV_MERGE_ROWS(__nv_bfloat16); break;
      case XKV_F16: XKV_MERGE_ROWS(__half); break;
      default: return XKV_ERR_BAD_ARG;
    }
#undef XKV_MERGE_ROWS
    return cudaGetLastError() == cudaSuccess ? XKV_OK : XKV_ERR_LAUNCH;
  }
  const size_t smem = (size_t)(num_splits + acc_dim) * sizeof(float);
  if (smem > 40 * 1024) return XKV_ERR_UNSUPPORTED;
  const dim3 grid(num_heads, batch);
  const int div = v_proj ? num_heads / v_proj_heads : 1;
  // vectorised projection: contiguous value columns, 16-byte aligned rows, lanes that divide the CTA
  const int es = dtype == XKV_F32 ? 4 : 2, vec = 16 / es;
  int vec_proj = 0;
  if (v_proj && vp_sd == 1 && value_dim % vec == 0 && value_dim / vec <= NT && NT % (value_dim / vec) == 0 &&
      (reinterpret_cast<uintptr_t>(v_proj) & 15u) == 0 && (vp_sr * es) % 16 == 0 && (vp_sh * es) % 16 == 0 &&
      (vp_sb * es) % 16 == 0)
    vec_proj = 1;
#define XKV_MERGE(T)                                                                                  \
  merge_kernel<T><<<grid, NT, smem, st>>>(partial_o, lse, static_cast<T*>(out), num_heads, heads_total, \
                                          head_offset, num_splits,                                  \
                                          acc_dim, value_dim, static_cast<const T*>(v_proj), div, vp_sb, \
                                          vp_sh, vp_sr, vp_sd, o_sb, o_sh, vec_proj, lse_out, lse_sb)
  switch (dtype) {
    case XKV_F32: XKV_MERGE(float); break;
    case XKV_BF16: XKV_MERGE(__nv_bfloat16); break;
    case XKV_F16: XKV_MERGE(__half); break;
    default: return XKV_ERR_BAD_ARG;
  }
#undef XKV_MERGE
  return cudaGetLastError() == cudaSuccess ? XKV_OK : XKV_ERR_LAUNCH;
}

int launch_rope_table(float* cos_sin, int kv_len, int half, int pos_offset, float theta,
                      const float* inv_freq, cudaStream_t st) {
  const int64_t n = (int64_t)kv_len * half;
  if (n <= 0) return XKV_ERR_BAD_ARG;
  rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(reinterpret_cast<float2*>(cos_sin), kv_len,
                                                                 half, pos_offset, theta, inv_freq);
  return cudaGetLastError() == cudaSuccess ? XKV_OK : XKV_ERR_LAUNCH;
}

}  // namespace xkv
