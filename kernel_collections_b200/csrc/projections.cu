// Projections around a shared-latent decode, batched over the batch rows.
//
// With a projection matrix shared by the whole batch (MLA's W_uk / W_uv, a shared B_k / B_v), folding it
// into the query and applying it to the merged output are small GEMMs [batch x in] . [in x out] per head.
// Done row by row (one CTA per (head, batch row)) every CTA re-reads its head's matrix from L2: at batch
// 64 with 128 heads that is 1 GB of L2 traffic per call on each side, more than the cache the attention
// itself streams.  Here one CTA owns a 128-column strip of one head's matrix and walks the batch in
// chunks, so the matrix is read once per chunk of 16 rows (grid: strips x heads x batch chunks).
#include "xkv_internal.h"

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
  const dim3 grid((unsigned)ceil_div(p.k_rank, NT), (unsigned)p.num_heads, (unsigned)ceil_div(p.batch, BC));
  // w[h/div, i = d, c = r] = k_proj[(h/div) * kp_sh + r * kp_sr + d * kp_sd]
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
int launch_value_projection_batched(const float* o_lat, const xkv_decode_params& p, cudaStream_t st) {
  const int div = p.num_heads / p.v_proj_heads;
  const dim3 grid((unsigned)ceil_div(p.value_dim, NT), (unsigned)p.num_heads, (unsigned)ceil_div(p.batch, BC));
  const size_t smem = (size_t)BC * p.v_rank * sizeof(float);
  const int64_t l_sb = (int64_t)p.num_heads * p.v_rank, l_sh = p.v_rank;
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
