// Per-step state around a decode call: rotating the new token's query to its position and
// projecting the new token's key (or value) row into latent space and appending it to the cache.
// Both are tiny next to the attention call (one row per sequence); they exist so that a decode
// step needs no eager tensor ops between kernels.
#include "xkv_internal.h"

namespace xkv {
namespace {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

// out[b, h, :] = x * cos + rotate_half(x) * sin at angle float(pos_b) * inv_freq[j]: the half-split
// rotation with pairs (j, j + D/2).  Products and the sum are rounded separately (no fused
// multiply-add) and cos / sin are the full-range library functions, so the result has the bits of
// the same expression evaluated with tensor ops.
template <typename T>
__global__ void rope_query_kernel(const T* __restrict__ q, T* __restrict__ out, int64_t q_sb, int64_t q_sh,
                                  int64_t o_sb, int64_t o_sh, int num_heads, int half, int position,
                                  const int32_t* __restrict__ positions, float theta,
                                  const float* __restrict__ inv_freq) {
  const int b = blockIdx.y;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= num_heads * half) return;
  const int h = idx / half, j = idx - h * half;
  const int pos = positions ? positions[b] : position;
  const float f = inv_freq ? inv_freq[j] : 1.0f / powf(theta, (float)(2 * j) / (float)(2 * half));
  const float ang = __fmul_rn((float)pos, f);
  const float cs = cosf(ang), sn = sinf(ang);
  const T* qr = q + (int64_t)b * q_sb + (int64_t)h * q_sh;
  T* orow = out + (int64_t)b * o_sb + (int64_t)h * o_sh;
  const float x0 = to_f(qr[j]), x1 = to_f(qr[j + half]);
  orow[j] = from_f<T>(__fadd_rn(__fmul_rn(x0, cs), __fmul_rn(-x1, sn)));
  orow[j + half] = from_f<T>(__fadd_rn(__fmul_rn(x1, cs), __fmul_rn(x0, sn)));
}

// latent[b, pos_b, r] = sum_c x[b, c] * proj[c, r]: one new cache row per sequence.  A block owns 128
// latent columns of one sequence; x is staged in shared memory as fp32, proj rows are read with the
// column index fastest (coalesced when the columns are contiguous), accumulation in fp32.
template <typename T>
__global__ void latent_append_kernel(const T* __restrict__ x, int64_t x_sb, const T* __restrict__ proj,
                                     int64_t p_sc, int64_t p_sr, T* __restrict__ latent, int64_t l_sb,
                                     int64_t l_sl, const int32_t* __restrict__ positions, int position,
                                     int in_dim, int rank, int capacity) {
  extern __shared__ float x_s[];
  const int b = blockIdx.y;
  const int pos = positions ? positions[b] : position;
  if (pos < 0 || pos >= capacity) return;   // a full (or idle) sequence appends nothing
  for (int c = threadIdx.x; c < in_dim; c += blockDim.x) x_s[c] = to_f(x[(int64_t)b * x_sb + c]);
  __syncthreads();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rank) return;
  const T* pr = proj + (int64_t)r * p_sr;
  float acc0 = 0.f, acc1 = 0.f;
  int c = 0;
  for (; c + 1 < in_dim; c += 2) {
    acc0 = fmaf(x_s[c], to_f(pr[(int64_t)c * p_sc]), acc0);
    acc1 = fmaf(x_s[c + 1], to_f(pr[(int64_t)(c + 1) * p_sc]), acc1);
  }
  if (c < in_dim) acc0 = fmaf(x_s[c], to_f(pr[(int64_t)c * p_sc]), acc0);
  latent[(int64_t)b * l_sb + (int64_t)pos * l_sl + r] = from_f<T>(acc0 + acc1);
}

}  // namespace

int launch_rope_query(const void* q, void* out, int dtype, int batch, int num_heads, int head_dim, int64_t q_sb,
                      int64_t q_sh, int64_t o_sb, int64_t o_sh, int position, const int32_t* positions, float theta,
                      const float* inv_freq, cudaStream_t st) {
  const int half = head_dim / 2;
  const dim3 grid((unsigned)ceil_div(num_heads * half, 128), (unsigned)batch);
#define XKV_RQ(T)                                                                                                  \
  rope_query_kernel<T><<<grid, 128, 0, st>>>(static_cast<const T*>(q), static_cast<T*>(out), q_sb, q_sh, o_sb, o_sh, \
                                             num_heads, half, position, positions, theta, inv_freq)
  switch (dtype) {
    case XKV_F32: XKV_RQ(float); break;
    case XKV_BF16: XKV_RQ(__nv_bfloat16); break;
    case XKV_F16: XKV_RQ(__half); break;
    default: return XKV_ERR_BAD_ARG;
  }
#undef XKV_RQ
  return cudaGetLastError() == cudaSuccess ? XKV_OK : XKV_ERR_LAUNCH;
}

int launch_latent_append(const void* x, int64_t x_sb, const void* proj, int64_t p_sc, int64_t p_sr, void* latent,
                         int64_t l_sb, int64_t l_sl, const int32_t* positions, int position, int dtype, int batch,
                         int in_dim, int rank, int capacity, cudaStream_t st) {
  const size_t smem = (size_t)in_dim * sizeof(float);
  if (smem > 48 * 1024) return XKV_ERR_UNSUPPORTED;
  const dim3 grid((unsigned)ceil_div(rank, 128), (unsigned)batch);
#define XKV_LA(T)                                                                                              \
  latent_append_kernel<T><<<grid, 128, smem, st>>>(static_cast<const T*>(x), x_sb, static_cast<const T*>(proj), \
                                                   p_sc, p_sr, static_cast<T*>(latent), l_sb, l_sl, positions, \
                                                   position, in_dim, rank, capacity)
  switch (dtype) {
    case XKV_F32: XKV_LA(float); break;
    case XKV_BF16: XKV_LA(__nv_bfloat16); break;
    case XKV_F16: XKV_LA(__half); break;
    default: return XKV_ERR_BAD_ARG;
  }
#undef XKV_LA
  return cudaGetLastError() == cudaSuccess ? XKV_OK : XKV_ERR_LAUNCH;
}

}  // namespace xkv
