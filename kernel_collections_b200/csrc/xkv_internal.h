// Internal declarations shared by the translation units of libxkv.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>
#include "xkv.h"

namespace xkv {

constexpr int kNumSMsFallback = 148;

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int elem_size(int dtype) { return dtype == XKV_F32 ? 4 : 2; }

int device_sm_count();

// ---- portable CUDA-core path (generic_decode.cu) -------------------------------------------
struct GenericPlan {
  int heads_per_cta;   // query heads handled by one CTA (divides the GQA group size)
  int head_chunks;     // num_heads / heads_per_cta
  int num_splits;      // KV splits
  int split_len;       // tokens per split (multiple of the token tile)
  int score_dim;       // width of the (effective) query / key rows
  int acc_dim;         // width of the accumulated value rows
  size_t off_qeff, off_partial, off_lse, total_bytes;
  size_t smem_bytes;
};
bool generic_plan(const xkv_decode_params& p, GenericPlan* plan);
int generic_decode(const xkv_decode_params& p, const GenericPlan& plan, void* ws, cudaStream_t st);
int generic_decode_builtin_scratch(const xkv_decode_params& p, const GenericPlan& plan, cudaStream_t st);
int launch_merge(const float* partial_o, const float* lse, void* out, int dtype, int batch,
                 int num_heads, int num_splits, int acc_dim, int value_dim, const void* v_proj,
                 int v_proj_heads, int64_t vp_sb, int64_t vp_sh, int64_t vp_sr, int64_t vp_sd,
                 int64_t o_sb, int64_t o_sh, cudaStream_t st, int heads_total = 0, int head_offset = 0,
                 float* lse_out = nullptr, int64_t lse_sb = 0);
int launch_rope_table(float* cos_sin, int kv_len, int half, int pos_offset, float theta,
                      const float* inv_freq, cudaStream_t st);

// ---- per-step state kernels (step_state.cu) ----------------------------------------------------
int launch_rope_query(const void* q, void* out, int dtype, int batch, int num_heads, int head_dim, int64_t q_sb,
                      int64_t q_sh, int64_t o_sb, int64_t o_sh, int position, const int32_t* positions, float theta,
                      const float* inv_freq, cudaStream_t st);
int launch_latent_append(const void* x, int64_t x_sb, const void* proj, int64_t p_sc, int64_t p_sr, void* latent,
                         int64_t l_sb, int64_t l_sl, const int32_t* positions, int position, int dtype, int batch,
                         int in_dim, int rank, int capacity, cudaStream_t st);

// ---- tcgen05 key-reconstruction path (recon_tc_sm100.cu) ------------------------------------
struct ReconTcPlan {
  int pair;             // CTA pairs (cta_group::2) instead of single CTAs
  int num_splits;       // CTAs (or CTA pairs) per batch row
  int tiles_per_split;  // 128-token tiles per CTA
  size_t off_partial, off_lse, total_bytes;
};
bool recon_tc_supported(const xkv_decode_params& p);
bool recon_tc_plan(const xkv_decode_params& p, ReconTcPlan* plan);
int recon_tc_decode(const xkv_decode_params& p, const ReconTcPlan& plan, void* ws, cudaStream_t st);
// one launch for the layers of a cross-layer group that share the key latent
bool recon_tc_group_supported(const xkv_decode_params* layers, int n);
bool recon_tc_group_plan(const xkv_decode_params* layers, int n, ReconTcPlan* plan);
// fp32 logits of a first pass: logits[layer * layer + b * sb + h * sh + token]
struct LogitsSink {
  float* ptr;
  int64_t sb, sh, layer;
};
int recon_tc_group_decode(const xkv_decode_params* layers, int n, const ReconTcPlan& plan, void* ws,
                          cudaStream_t st, const LogitsSink* sink);
bool recon_tc_logits_supported(const xkv_decode_params* layers, int n);
bool recon_tc_logits_plan(const xkv_decode_params* layers, int n, ReconTcPlan* plan);

// ---- dense GQA decode on mma.sync + TMA (dense_tc_sm100.cu) ----------------------------------
struct DenseTcPlan {
  int num_splits, tiles;
  size_t off_partial, off_lse, total_bytes;
};
bool dense_tc_supported(const xkv_decode_params& p);
bool dense_tc_plan(const xkv_decode_params& p, DenseTcPlan* plan);
struct LogitsSink;
bool dense_tc_logits_supported(const xkv_decode_params& p);
int dense_tc_decode(const xkv_decode_params& p, const DenseTcPlan& plan, void* ws, cudaStream_t st,
                    const LogitsSink* sink = nullptr);
// second pass for keys that are not dense: softmax over fp32 logits, P.V with dense values
bool dense_tc_values_supported(const xkv_decode_params& p);
int dense_tc_values_from_logits(const xkv_decode_params& p, const DenseTcPlan& plan, const LogitsSink& logits, void* ws,
                                int* status, cudaStream_t st);

// ---- shared-latent decode (absorbed factorized K / V, MLA) on mma.sync + TMA (latent_tc_sm100.cu)
struct LatentTcPlan {
  int heads_per_cta, stages, num_splits, tiles;
  size_t smem_bytes;
  size_t off_qeff, off_partial, off_lse, total_bytes;
  size_t off_olat;     // fp32 merged latent rows in front of a batched value projection (0: unused)
};
bool latent_tc_supported(const xkv_decode_params& p);
bool latent_tc_plan(const xkv_decode_params& p, LatentTcPlan* plan);
int latent_tc_decode(const xkv_decode_params& p, const LatentTcPlan& plan, void* ws, cudaStream_t st,
                     const LogitsSink* sink = nullptr);
// second pass of a two-pass decode: softmax over fp32 logits of `heads` stacked heads, times the value latent
bool latent_pv_supported(const xkv_decode_params& p);
bool latent_pv_plan(const xkv_decode_params& p, int heads, LatentTcPlan* plan);
int latent_pv_run(const xkv_decode_params& p, int heads, const LatentTcPlan& plan, const float* logits, void* ws,
                  int* status, cudaStream_t st);

// prologue shared by the shared-latent kernels: q_eff[b, h, :] = q . k_proj^T (or q) | q_tail, in the working dtype
int launch_absorb_query_lowp(const xkv_decode_params& p, void* qeff, int dk, cudaStream_t st);

// projections batched over the batch rows, for matrices shared by the batch (projections.cu)
bool batched_projection_fits(int batch, int in_dim);
int launch_absorb_query_batched(const xkv_decode_params& p, void* qeff, int dk, cudaStream_t st);
// `lse` / `num_splits` > 1: o_lat holds per-split partial rows [batch][heads][splits][v_rank] with their log-sum-exps
// [batch][heads][splits], merged while they are staged (value_projection_merges says whether this call can do that)
int launch_value_projection_batched(const float* o_lat, const xkv_decode_params& p, cudaStream_t st,
                                    const float* lse = nullptr, int num_splits = 1);
bool value_projection_merges(const xkv_decode_params& p, int num_splits);

// ---- shared-latent decode on tcgen05, two CTAs per tile (latent_pair_sm100.cu) -------------------
bool latent_pair_supported(const xkv_decode_params& p);
bool latent_pair_plan(const xkv_decode_params& p, LatentTcPlan* plan);
int latent_pair_decode(const xkv_decode_params& p, const LatentTcPlan& plan, void* ws, cudaStream_t st);

// ---- tcgen05 softmax + P.A_v pass with the output in TMEM (pv_tc_sm100.cu) ------------------------
struct PvTcPlan {
  int col_blocks, head_blocks, tiles, num_splits;
  size_t off_partial, off_lse, total_bytes;
};
bool pv_tc_supported(const xkv_decode_params& p);
bool pv_tc_plan(const xkv_decode_params& p, int heads, PvTcPlan* plan);
int pv_tc_run(const xkv_decode_params& p, int heads, const PvTcPlan& plan, const float* logits, void* ws,
              int* status, cudaStream_t st);

// ---- two-pass decode for factorized values behind dense / RoPE-reconstructed keys (two_pass.cu)
struct TwoPassPlan {
  int dense_values;          // 1: absorbed factorized keys (no RoPE) in front of dense values
  LatentTcPlan klat;         //    first pass: shared-latent kernel, logits only
  DenseTcPlan vdense;        //    second pass: dense kernel, scores from logits
  int heads;                 // layers x heads, stacked for the second pass
  ReconTcPlan recon;
  DenseTcPlan dense;
  LatentTcPlan pv;           // second pass on mma.sync (XKV_PV_MMA_SYNC=1), or
  PvTcPlan pv_tc;            // on tcgen05 with the output in TMEM
  int use_pv_tc;
  size_t off_logits, off_pass1, off_pass2, total_bytes;
};
bool two_pass_supported(const xkv_decode_params* layers, int n);
bool two_pass_plan(const xkv_decode_params* layers, int n, TwoPassPlan* plan);
int two_pass_decode(const xkv_decode_params* layers, int n, const TwoPassPlan& plan, void* ws, cudaStream_t st);

}  // namespace xkv
