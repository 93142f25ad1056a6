// Projections around a shared-latent decode, batched over the batch rows.
//
// With a projection matrix shared by the whole batch (MLA's W_uk / W_uv, a shared B_k / B_v), folding it
// into the query and applying it to the merged output are small GEMMs [batch x in] . [in x out] per head.
// Done row by row (one CTA per (head, batch row)) every CTA re-reads its head's matrix from L2: at batch
// 64 with 128 heads that is 1 GB of L2 traffic per call on each side, more than the cache the attention
// itself streams.  Here one CTA owns a 128-column strip of one head's matrix and walks the batch in
// chunks, so the matrix is read once per chunk of 16 rows (grid: strips x heads x batch chunks).
#include "sm100_common.cuh"

namespace xkv {
namespace {

constexpr int BC = 16;          // batch rows per chunk (accumulators per thread)
constexpr int NT = 128;         // threads per CTA = output columns per CTA

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

// out[b, h, c] = sum_i x[b, h, i] * w[h / div, i, c] for c in this CTA's strip, all b.
// x: TI elements at x + b * x_sb + h * x_sh (contiguous in i); w addressed as w + (h / div) * w_sh + i * w_si + c * w_sc;
// out: TO elements at out + b * o_sb + h * o_sh + c.
template <typename TI, typename TW, typename TO>
__global__ void __launch_bounds__(NT)
batched_projection_kernel(const TI* __restrict__ x, int64_t x_sb, int64_t x_sh, const TW* __restrict__ w, int div,
                          int64_t w_sh, int64_t w_si, int64_t w_sc, TO* __restrict__ out, int64_t o_sb, int64_t o_sh,
                          int batch, int in_dim, int out_dim) {
  extern __shared__ float x_s[];                 // [in_dim][BC]: the chunk's rows, batch index fastest
  const int h = blockIdx.y;
  const int c = blockIdx.x * NT + threadIdx.x;
  const int b0 = blockIdx.z * BC;
  const int nb = min(BC, batch - b0);
  for (int idx = threadIdx.x; idx < BC * in_dim; idx += NT) {
    const int j = idx / in_dim, i = idx - j * in_dim;
    x_s[i * BC + j] = j < nb ? to_f(x[(int64_t)(b0 + j) * x_sb + (int64_t)h * x_sh + i]) : 0.f;
  }
  __syncthreads();
  if (c >= out_dim) return;
  const TW* wc = w + (int64_t)(h / div) * w_sh + (int64_t)c * w_sc;
  float acc[BC];
#pragma unroll
  for (int j = 0; j < BC; ++j) acc[j] = 0.f;
  // the matrix column is walked 16 rows at a time: 16 independent loads in flight per thread cover the L2 latency
  constexpr int UI = 16;
  for (int i0 = 0; i0 < in_dim; i0 += UI) {
    float wv[UI];
#pragma unroll
    for (int u = 0; u < UI; ++u) wv[u] = (i0 + u < in_dim) ? to_f(wc[(int64_t)(i0 + u) * w_si]) : 0.f;
#pragma unroll
    for (int u = 0; u < UI; ++u) {
      if (i0 + u < in_dim) {
        const float4* xr = reinterpret_cast<const float4*>(x_s + (i0 + u) * BC);
#pragma unroll
        for (int j4 = 0; j4 < BC / 4; ++j4) {
          const float4 xv = xr[j4];
          acc[4 * j4] = fmaf(xv.x, wv[u], acc[4 * j4]);
          acc[4 * j4 + 1] = fmaf(xv.y, wv[u], acc[4 * j4 + 1]);
          acc[4 * j4 + 2] = fmaf(xv.z, wv[u], acc[4 * j4 + 2]);
          acc[4 * j4 + 3] = fmaf(xv.w, wv[u], acc[4 * j4 + 3]);
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < BC; ++j)
    if (j < nb) out[(int64_t)(b0 + j) * o_sb + (int64_t)h * o_sh + c] = from_f<TO>(acc[j]);
}

// ---- the same product on the tensor cores (mma.sync m16n8k16, fp32 accumulation) -------------------------------
// One CTA of four warps owns, for one head, a tile of MM = 64 batch rows x MN = 64 output columns and walks the
// contraction in chunks of MK = 64: the chunk of x and of the head's matrix are staged in shared memory as 16-bit
// values, warp w multiplies rows 16 w .. 16 w + 15.  fp32 inputs (merged latent rows) are split into a rounded
// 16-bit value and the 16-bit remainder and multiplied twice, so the product keeps the input's precision.
// W_K says which index of the matrix is contiguous in memory: the contraction index (w_si == 1) or the output column
// (w_sc == 1).  Rows of a strip past `batch` are zero.  `tail`: the absorbed query's pass-through columns, copied
// by the CTAs of strip 0.
constexpr int MM = 64, MN = 64, MK = 64, MPAD = 8;
constexpr int MERGE_MAX = 16;     // most splits the fp32 staging merges on the way

template <typename TI, typename T, bool W_K>
__global__ void __launch_bounds__(128)
projection_mma_kernel(const TI* __restrict__ x, int64_t x_sb, int64_t x_sh, const T* __restrict__ w, int div, int64_t w_sh,
                      int64_t w_si, int64_t w_sc, T* __restrict__ out, int64_t o_sb, int64_t o_sh, int batch, int in_dim,
                      int out_dim, const T* __restrict__ tail, int64_t t_sb, int64_t t_sh, int tail_dim, int tail_col,
                      const float* __restrict__ lse, int nsplit) {
  constexpr bool SPLIT = sizeof(TI) == 4;
  __shared__ float wsp[SPLIT ? MM : 1][SPLIT ? MERGE_MAX : 1];   // merge weights of the strip's rows
  __shared__ __align__(16) T xs[SPLIT ? 2 : 1][MM][MK + MPAD];
  __shared__ __align__(16) T ws[MK][MN + MPAD];            // W_K: [column][contraction], else [contraction][column]
  const int h = blockIdx.y, c0 = blockIdx.x * MN, b0 = blockIdx.z * MM;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const T* wh = w + (int64_t)(h / div) * w_sh;
  if (tail != nullptr && blockIdx.x == 0) {
    // (the launcher has checked: tail_dim a multiple of 8, 16-byte aligned rows on both sides)
    const int per_row = tail_dim / 8;
    for (int idx = threadIdx.x; idx < MM * per_row; idx += 128) {
      const int j = idx / per_row, d = (idx - j * per_row) * 8;
      if (b0 + j < batch)
        *reinterpret_cast<uint4*>(out + (int64_t)(b0 + j) * o_sb + (int64_t)h * o_sh + tail_col + d) =
            *reinterpret_cast<const uint4*>(tail + (int64_t)(b0 + j) * t_sb + (int64_t)h * t_sh + d);
    }
  }
  float acc[MN / 8][4];
#pragma unroll
  for (int n = 0; n < MN / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;
  if constexpr (SPLIT) {
    // x given as per-split partial rows (each normalised) and their log-sum-exps: the merged row is their
    // combination with weights exp(lse_s - max) / sum; an empty split has lse = -inf and weight 0
    if (nsplit > 1 && threadIdx.x < MM) {
      const int j = threadIdx.x;
      float l[MERGE_MAX], mx = -CUDART_INF_F, sum = 0.f;
      for (int sidx = 0; sidx < nsplit; ++sidx) {
        l[sidx] = b0 + j < batch ? lse[((int64_t)(b0 + j) * gridDim.y + h) * nsplit + sidx] : -CUDART_INF_F;
        mx = fmaxf(mx, l[sidx]);
      }
      for (int sidx = 0; sidx < nsplit; ++sidx) {
        l[sidx] = mx == -CUDART_INF_F ? 0.f : __expf(l[sidx] - mx);
        sum += l[sidx];
      }
      for (int sidx = 0; sidx < nsplit; ++sidx) wsp[j][sidx] = sum > 0.f ? l[sidx] / sum : 0.f;
    }
  }

  // Software pipeline: the next chunk's global loads are issued into registers before the current chunk's MMAs,
  // so a chunk costs the longer of the two, not their sum (the CTAs are too few to hide the latency by themselves).
  constexpr int XI = MM * (MK / 8) / 128;      // 16-byte (8-value) pieces of x per thread and chunk
  constexpr int WI = MK * (MN / 8) / 128;      // 16-byte pieces of the matrix per thread and chunk
  float4 xr[SPLIT ? XI : 1][2];
  uint4 xr16[SPLIT ? 1 : XI];
  uint4 wr[WI];
  (void)xr; (void)xr16;
  auto fetch = [&](int k0) {
#pragma unroll
    for (int it = 0; it < XI; ++it) {
      const int idx = threadIdx.x + it * 128;
      const int j = idx / (MK / 8), k8 = (idx - j * (MK / 8)) * 8;
      const TI* src = x + (int64_t)(b0 + j) * x_sb + (int64_t)h * x_sh + k0 + k8;
      if constexpr (SPLIT) {
        float4 f0 = make_float4(0.f, 0.f, 0.f, 0.f), f1 = f0;
        if (b0 + j < batch) {
          f0 = *reinterpret_cast<const float4*>(src);
          f1 = *reinterpret_cast<const float4*>(src + 4);
          if (nsplit > 1) {
            const float w0 = wsp[j][0];
            f0 = make_float4(f0.x * w0, f0.y * w0, f0.z * w0, f0.w * w0);
            f1 = make_float4(f1.x * w0, f1.y * w0, f1.z * w0, f1.w * w0);
            for (int sidx = 1; sidx < nsplit; ++sidx) {
              const float wv = wsp[j][sidx];
              const float4 g0 = *reinterpret_cast<const float4*>(src + (int64_t)sidx * in_dim);
              const float4 g1 = *reinterpret_cast<const float4*>(src + (int64_t)sidx * in_dim + 4);
              f0 = make_float4(fmaf(g0.x, wv, f0.x), fmaf(g0.y, wv, f0.y), fmaf(g0.z, wv, f0.z), fmaf(g0.w, wv, f0.w));
              f1 = make_float4(fmaf(g1.x, wv, f1.x), fmaf(g1.y, wv, f1.y), fmaf(g1.z, wv, f1.z), fmaf(g1.w, wv, f1.w));
            }
          }
        }
        xr[it][0] = f0;
        xr[it][1] = f1;
      } else {
        xr16[it] = b0 + j < batch ? *reinterpret_cast<const uint4*>(src) : make_uint4(0u, 0u, 0u, 0u);
      }
    }
#pragma unroll
    for (int it = 0; it < WI; ++it) {
      const int idx = threadIdx.x + it * 128;
      const int r = idx / 8, q8 = (idx & 7) * 8;
      const T* src = W_K ? wh + (int64_t)(c0 + r) * w_sc + (k0 + q8) : wh + (int64_t)(k0 + r) * w_si + (c0 + q8);
      wr[it] = *reinterpret_cast<const uint4*>(src);
    }
  };
  auto stage = [&]() {
#pragma unroll
    for (int it = 0; it < XI; ++it) {
      const int idx = threadIdx.x + it * 128;
      const int j = idx / (MK / 8), k8 = (idx - j * (MK / 8)) * 8;
      if constexpr (SPLIT) {
        const float f[8] = {xr[it][0].x, xr[it][0].y, xr[it][0].z, xr[it][0].w, xr[it][1].x, xr[it][1].y, xr[it][1].z, xr[it][1].w};
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          hi[e] = sm100::TypeTraits<T>::pack2(f[2 * e], f[2 * e + 1]);
          const float2 back = sm100::TypeTraits<T>::unpack2(hi[e]);
          lo[e] = sm100::TypeTraits<T>::pack2(f[2 * e] - back.x, f[2 * e + 1] - back.y);
        }
        *reinterpret_cast<uint4*>(&xs[0][j][k8]) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(&xs[SPLIT ? 1 : 0][j][k8]) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      } else {
        *reinterpret_cast<uint4*>(&xs[0][j][k8]) = xr16[it];
      }
    }
#pragma unroll
    for (int it = 0; it < WI; ++it) {
      const int idx = threadIdx.x + it * 128;
      *reinterpret_cast<uint4*>(&ws[idx / 8][(idx & 7) * 8]) = wr[it];
    }
  };

  __syncthreads();                               // the merge weights are in place
  fetch(0);
  for (int k0 = 0; k0 < in_dim; k0 += MK) {
    if (k0 > 0) __syncthreads();                 // the previous chunk's MMAs have read their operands
    stage();
    __syncthreads();
    if (k0 + MK < in_dim) fetch(k0 + MK);
#pragma unroll
    for (int kk = 0; kk < MK; kk += 16) {
      uint32_t a[SPLIT ? 2 : 1][4];
#pragma unroll
      for (int part = 0; part < (SPLIT ? 2 : 1); ++part) {
        a[part][0] = *reinterpret_cast<const uint32_t*>(&xs[part][warp * 16 + g][kk + 2 * t]);
        a[part][1] = *reinterpret_cast<const uint32_t*>(&xs[part][warp * 16 + g + 8][kk + 2 * t]);
        a[part][2] = *reinterpret_cast<const uint32_t*>(&xs[part][warp * 16 + g][kk + 2 * t + 8]);
        a[part][3] = *reinterpret_cast<const uint32_t*>(&xs[part][warp * 16 + g + 8][kk + 2 * t + 8]);
      }
#pragma unroll
      for (int n = 0; n < MN / 8; ++n) {
        uint32_t b0r, b1r;
        if constexpr (W_K) {
          b0r = *reinterpret_cast<const uint32_t*>(&ws[n * 8 + g][kk + 2 * t]);
          b1r = *reinterpret_cast<const uint32_t*>(&ws[n * 8 + g][kk + 2 * t + 8]);
        } else {
          // rows of ws are contraction indices: the transposing matrix load hands every thread its (k, k + 1) pairs
          const uint32_t addr = sm100::smem_u32(&ws[kk + (lane & 15)][n * 8]);
          asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(b0r), "=r"(b1r) : "r"(addr));
        }
#pragma unroll
        for (int part = 0; part < (SPLIT ? 2 : 1); ++part) sm100::TypeTraits<T>::mma(acc[n], a[part], b0r, b1r);
      }
    }
  }
  const int r0 = b0 + warp * 16 + g;
#pragma unroll
  for (int n = 0; n < MN / 8; ++n) {
    const int c = c0 + n * 8 + 2 * t;
    if (c >= out_dim) continue;
    // (c is even and the launcher has checked that rows start on 4-byte boundaries: one store per pair)
    T* o0 = out + (int64_t)r0 * o_sb + (int64_t)h * o_sh + c;
    T* o1 = out + (int64_t)(r0 + 8) * o_sb + (int64_t)h * o_sh + c;
    if (r0 < batch) *reinterpret_cast<uint32_t*>(o0) = sm100::TypeTraits<T>::pack2(acc[n][0], acc[n][1]);
    if (r0 + 8 < batch) *reinterpret_cast<uint32_t*>(o1) = sm100::TypeTraits<T>::pack2(acc[n][2], acc[n][3]);
  }
}

// Whether the tensor-core kernel can take a product: whole 64-wide chunks, one contiguous matrix index, 16-byte
// aligned rows everywhere it loads 16 bytes at a time.
template <typename TI>
bool projection_mma_ok(const void* x, int64_t x_sb, int64_t x_sh, const void* w, int64_t w_sh, int64_t w_si, int64_t w_sc,
                       int in_dim, int out_dim) {
  const int xa = 16 / (int)sizeof(TI);
  if (in_dim % MK != 0 || out_dim % MN != 0) return false;
  if (!sm100::aligned16(x) || x_sb % xa != 0 || x_sh % xa != 0) return false;
  if (!sm100::aligned16(w) || w_sh % 8 != 0) return false;
  if (w_si == 1) return w_sc % 8 == 0;
  if (w_sc == 1) return w_si % 8 == 0;
  return false;
}

template <typename T>
__global__ void copy_tail_kernel(const T* __restrict__ qt, int64_t qt_sb, int64_t qt_sh, T* __restrict__ out, int dk,
                                 int k_rank, int tail, int num_heads) {
  const int h = blockIdx.x, b = blockIdx.y;
  for (int d = threadIdx.x; d < tail; d += blockDim.x)
    out[((int64_t)b * num_heads + h) * dk + k_rank + d] = qt[(int64_t)b * qt_sb + (int64_t)h * qt_sh + d];
}

}  // namespace

bool batched_projection_fits(int batch, int in_dim) {
  return batch >= 4 && (size_t)BC * in_dim * sizeof(float) <= 48 * 1024;
}

// q_eff[b, h, 0:k_rank] = q[b, h, :] . k_proj[h / div]^T and q_eff[b, h, k_rank:] = q_tail[b, h, :], working dtype.
// Requires a projection shared by the batch (kp_sb == 0) and batched_projection_fits(batch, head_dim).
template <typename T>
static int absorb_batched(const xkv_decode_params& p, T* qeff, int dk, cudaStream_t st) {
  const int div = p.num_heads / p.k_proj_heads;
  // w[h/div, i = d, c = r] = k_proj[(h/div) * kp_sh + r * kp_sr + d * kp_sd]
  if (projection_mma_ok<T>(p.q, p.q_sb, p.q_sh, p.k_proj, p.kp_sh, p.kp_sd, p.kp_sr, p.head_dim, p.k_rank) && dk % 2 == 0 &&
      (reinterpret_cast<uintptr_t>(qeff) & 3u) == 0 &&
      (p.tail_dim == 0 || (p.q_tail != nullptr && p.tail_dim % 8 == 0 && dk % 8 == 0 && p.k_rank % 8 == 0 &&
                           sm100::aligned16(p.q_tail) && p.qt_sb % 8 == 0 && p.qt_sh % 8 == 0 && sm100::aligned16(qeff)))) {
    const dim3 mgrid((unsigned)(p.k_rank / MN), (unsigned)p.num_heads, (unsigned)ceil_div(p.batch, MM));
    const T* tail = p.tail_dim > 0 ? static_cast<const T*>(p.q_tail) : nullptr;
    if (p.kp_sd == 1)
      projection_mma_kernel<T, T, true><<<mgrid, 128, 0, st>>>(static_cast<const T*>(p.q), p.q_sb, p.q_sh,
          static_cast<const T*>(p.k_proj), div, p.kp_sh, p.kp_sd, p.kp_sr, qeff, (int64_t)p.num_heads * dk, (int64_t)dk, p.batch,
          p.head_dim, p.k_rank, tail, p.qt_sb, p.qt_sh, p.tail_dim, p.k_rank, nullptr, 1);
    else
      projection_mma_kernel<T, T, false><<<mgrid, 128, 0, st>>>(static_cast<const T*>(p.q), p.q_sb, p.q_sh,
          static_cast<const T*>(p.k_proj), div, p.kp_sh, p.kp_sd, p.kp_sr, qeff, (int64_t)p.num_heads * dk, (int64_t)dk, p.batch,
          p.head_dim, p.k_rank, tail, p.qt_sb, p.qt_sh, p.tail_dim, p.k_rank, nullptr, 1);
    return cudaGetLastError() == cudaSuccess ? XKV_OK : XKV_ERR_LAUNCH;
  }
  const dim3 grid((unsigned)ceil_div(p.k_rank, NT), (unsigned)p.num_heads, (unsigned)ceil_div(p.batch, BC));
  batched_projection_kernel<T, T, T><<<grid, NT, (size_t)BC * p.head_dim * sizeof(float), st>>>(
      static_cast<const T*>(p.q), p.q_sb, p.q_sh, static_cast<const T*>(p.k_proj), div, p.kp_sh, p.kp_sd, p.kp_sr, qeff,
      (int64_t)p.num_heads * dk, (int64_t)dk, p.batch, p.head_dim, p.k_rank);
  if (p.tail_dim > 0)
    copy_tail_kernel<T><<<dim3(p.num_heads, p.batch), 64, 0, st>>>(static_cast<const T*>(p.q_tail), p.qt_sb, p.qt_sh, qeff, dk,
                                                                   p.k_rank, p.tail_dim, p.num_heads);
  return cudaGetLastError() == cudaSuccess ? XKV_OK : XKV_ERR_LAUNCH;
}

int launch_absorb_query_batched(const xkv_decode_params& p, void* qeff, int dk, cudaStream_t st) {
  if (p.dtype == XKV_BF16) return absorb_batched(p, static_cast<__nv_bfloat16*>(qeff), dk, st);
  if (p.dtype == XKV_F16) return absorb_batched(p, static_cast<__half*>(qeff), dk, st);
  return XKV_ERR_UNSUPPORTED;
}

// out[b, h, :] = o_lat[b, h, :] . v_proj[h / div] (fp32 merged latent rows -> output dtype), shared projection.
static bool value_projection_mma_ok(const float* o_lat, const xkv_decode_params& p, int64_t l_sb, int64_t l_sh) {
  return (p.dtype == XKV_BF16 || p.dtype == XKV_F16) && p.o_sb % 2 == 0 && p.o_sh % 2 == 0 &&
         (reinterpret_cast<uintptr_t>(p.out) & 3u) == 0 &&
         projection_mma_ok<float>(o_lat, l_sb, l_sh, p.v_proj, p.vp_sh, p.vp_sr, p.vp_sd, p.v_rank, p.value_dim);
}

bool value_projection_merges(const xkv_decode_params& p, int num_splits) {
  if (num_splits < 1 || num_splits > MERGE_MAX || p.v_rank % 4 != 0) return false;
  // (the partial rows sit in the 256-byte aligned workspace: only the matrix and the output decide)
  return value_projection_mma_ok(nullptr, p, (int64_t)p.num_heads * num_splits * p.v_rank, (int64_t)num_splits * p.v_rank);
}

int launch_value_projection_batched(const float* o_lat, const xkv_decode_params& p, cudaStream_t st, const float* lse,
                                    int num_splits) {
  const int div = p.num_heads / p.v_proj_heads;
  if (num_splits > 1 && (lse == nullptr || !value_projection_merges(p, num_splits))) return XKV_ERR_UNSUPPORTED;
  const dim3 grid((unsigned)ceil_div(p.value_dim, NT), (unsigned)p.num_heads, (unsigned)ceil_div(p.batch, BC));
  const size_t smem = (size_t)BC * p.v_rank * sizeof(float);
  const int64_t l_sb = (int64_t)p.num_heads * num_splits * p.v_rank, l_sh = (int64_t)num_splits * p.v_rank;
  // w[h/div, i = r, c = d] = v_proj[(h/div) * vp_sh + r * vp_sr + d * vp_sd]
  if (value_projection_mma_ok(o_lat, p, l_sb, l_sh)) {
    const dim3 mgrid((unsigned)(p.value_dim / MN), (unsigned)p.num_heads, (unsigned)ceil_div(p.batch, MM));
#define XKV_VPM(T, WK)                                                                                                   \
  projection_mma_kernel<float, T, WK><<<mgrid, 128, 0, st>>>(o_lat, l_sb, l_sh, static_cast<const T*>(p.v_proj), div, p.vp_sh, \
      p.vp_sr, p.vp_sd, static_cast<T*>(p.out), p.o_sb, p.o_sh, p.batch, p.v_rank, p.value_dim, nullptr, 0, 0, 0, 0, lse, num_splits)
    if (p.dtype == XKV_BF16) { if (p.vp_sr == 1) XKV_VPM(__nv_bfloat16, true); else XKV_VPM(__nv_bfloat16, false); }
    else { if (p.vp_sr == 1) XKV_VPM(__half, true); else XKV_VPM(__half, false); }
#undef XKV_VPM
    return cudaGetLastError() == cudaSuccess ? XKV_OK : XKV_ERR_LAUNCH;
  }
#define XKV_VP(T)                                                                                                     \
  batched_projection_kernel<float, T, T><<<grid, NT, smem, st>>>(o_lat, l_sb, l_sh, static_cast<const T*>(p.v_proj), div, \
                                                                  p.vp_sh, p.vp_sr, p.vp_sd, static_cast<T*>(p.out), p.o_sb, \
                                                                  p.o_sh, p.batch, p.v_rank, p.value_dim)
  if (p.dtype == XKV_BF16) { XKV_VP(__nv_bfloat16); }
  else if (p.dtype == XKV_F16) { XKV_VP(__half); }
  else return XKV_ERR_UNSUPPORTED;
#undef XKV_VP
  return cudaGetLastError() == cudaSuccess ? XKV_OK : XKV_ERR_LAUNCH;
}

}  // namespace xkv
