// Two-pass decode for factorized values behind keys that are dense or rebuilt with RoPE.
//
// The tensor-core key kernels keep their P.V accumulators in registers, which rules out value rows
// of rank 256-1024 shared by every head.  Such calls run as two passes over one workspace:
//   pass 1  fp32 logits sm_scale * q.k for every (layer, head, token): the tcgen05 key
//           reconstruction kernel (all layers of a cross-layer group in one launch) or the dense
//           key kernel, both in their logits-only mode;
//   pass 2  softmax over the logits and P . A_v with the heads of all layers stacked on the M
//           dimension, so the shared value latent is streamed once for the whole group;
//   merge   per layer: log-sum-exp merge of the splits and that layer's B_v projection.
// The logits round trip costs 8 bytes per (head, token) of HBM traffic, a few percent of the latent
// rows it sits next to.
#include "xkv_internal.h"

namespace xkv {

namespace {
bool same_values(const xkv_decode_params& a, const xkv_decode_params& b) {
  return a.v == b.v && a.v_sb == b.v_sb && a.v_sl == b.v_sl && a.v_rank == b.v_rank && a.value_dim == b.value_dim &&
         a.batch == b.batch && a.kv_len == b.kv_len && a.num_heads == b.num_heads && a.dtype == b.dtype &&
         a.kv_lens == b.kv_lens;
}
}  // namespace

// Factorized keys without RoPE in front of dense values (the reference's `k_only` fused kernel):
// logits from the shared-latent kernel (absorbed order, the latent is streamed once), then softmax
// and P.V on the dense-value kernel.
static xkv_decode_params key_logits_call(const xkv_decode_params& p) {
  xkv_decode_params t = p;
  t.flags |= XKV_FLAG_LOGITS_ONLY;
  t.lg_sb = (int64_t)p.num_heads * p.kv_len;
  t.lg_sh = p.kv_len;
  return t;
}
static bool dense_values_supported(const xkv_decode_params& p) {
  if (p.score_mode != XKV_SCORE_LATENT || p.value_mode != XKV_VALUE_DENSE || p.tail_dim != 0 || !p.k_proj) return false;
  return dense_tc_values_supported(p) && latent_tc_supported(key_logits_call(p));
}

bool two_pass_supported(const xkv_decode_params* layers, int n) {
  if (n < 1 || n > 8) return false;
  const xkv_decode_params& p = layers[0];
  if (p.flags & (XKV_FLAG_FORCE_GENERIC | XKV_FLAG_LOGITS_ONLY)) return false;
  if (n == 1 && dense_values_supported(p)) return true;
  if (!latent_pv_supported(p)) return false;
  for (int i = 0; i < n; ++i) {
    if (!same_values(p, layers[i]) || layers[i].score_mode != p.score_mode) return false;
    if (layers[i].flags & (XKV_FLAG_FORCE_GENERIC | XKV_FLAG_LOGITS_ONLY)) return false;
  }
  if (p.score_mode == XKV_SCORE_RECON_ROPE) return recon_tc_logits_supported(layers, n);
  if (p.score_mode == XKV_SCORE_DENSE) {
    for (int i = 0; i < n; ++i)
      if (!dense_tc_logits_supported(layers[i])) return false;
    return true;
  }
  return false;
}

bool two_pass_plan(const xkv_decode_params* layers, int n, TwoPassPlan* pl) {
  const xkv_decode_params& p = layers[0];
  const int heads = n * p.num_heads;
  pl->heads = heads;
  pl->dense_values = (n == 1 && dense_values_supported(p)) ? 1 : 0;
  if (pl->dense_values) {
    if (!latent_tc_plan(key_logits_call(p), &pl->klat) || !dense_tc_plan(p, &pl->vdense)) return false;
    size_t off = 0;
    pl->off_pass1 = off;
    off += align_up(pl->klat.total_bytes, 256);
    pl->off_logits = off;
    off += align_up((size_t)p.batch * heads * p.kv_len * sizeof(float), 256);
    pl->off_pass2 = off;
    off += pl->vdense.total_bytes;
    pl->total_bytes = off;
    pl->use_pv_tc = 0;
    return true;
  }
  // the first pass's workspace leads, so that its status words are the ones the caller reads;
  // the second pass reports into the same words
  size_t off = 0;
  pl->off_pass1 = off;
  size_t p1 = 0;
  if (p.score_mode == XKV_SCORE_RECON_ROPE) {
    if (!recon_tc_logits_plan(layers, n, &pl->recon)) return false;
    p1 = pl->recon.total_bytes;
  } else {
    xkv_decode_params t = p;
    if (!dense_tc_plan(t, &pl->dense)) return false;
    p1 = pl->dense.total_bytes;
  }
  off += align_up(p1, 256);
  pl->off_logits = off;
  off += align_up((size_t)p.batch * heads * p.kv_len * sizeof(float), 256);
  pl->off_pass2 = off;
  // second pass: tcgen05 kernel with the output in TMEM; XKV_FLAG_PV_MMA_SYNC keeps the mma.sync one
  pl->use_pv_tc = (pv_tc_supported(p) && !(p.flags & XKV_FLAG_PV_MMA_SYNC)) ? 1 : 0;
  if (pl->use_pv_tc) {
    if (!pv_tc_plan(p, heads, &pl->pv_tc)) return false;
    off += pl->pv_tc.total_bytes;
  } else {
    if (!latent_pv_plan(p, heads, &pl->pv)) return false;
    off += pl->pv.total_bytes;
  }
  pl->total_bytes = off;
  return true;
}

int two_pass_decode(const xkv_decode_params* layers, int n, const TwoPassPlan& pl, void* ws, cudaStream_t st) {
  const xkv_decode_params& p = layers[0];
  char* w = static_cast<char*>(ws);
  float* logits = reinterpret_cast<float*>(w + pl.off_logits);
  const int H = p.num_heads, heads = pl.heads;
  LogitsSink sink{logits, (int64_t)heads * p.kv_len, (int64_t)p.kv_len, (int64_t)H * p.kv_len};
  int rc;
  if (pl.dense_values) {
    rc = latent_tc_decode(key_logits_call(p), pl.klat, w + pl.off_pass1, st, &sink);
    if (rc != XKV_OK) return rc;
    // the first pass cleared the status words at the head of the workspace; the second reports into them
    return dense_tc_values_from_logits(p, pl.vdense, sink, w + pl.off_pass2, reinterpret_cast<int*>(w), st);
  }
  if (p.score_mode == XKV_SCORE_RECON_ROPE) {
    rc = recon_tc_group_decode(layers, n, pl.recon, w + pl.off_pass1, st, &sink);
    if (rc != XKV_OK) return rc;
  } else {
    for (int i = 0; i < n; ++i) {
      LogitsSink si{logits + (int64_t)i * H * p.kv_len, sink.sb, sink.sh, 0};
      rc = dense_tc_decode(layers[i], pl.dense, w + pl.off_pass1, st, &si);
      if (rc != XKV_OK) return rc;
    }
  }
  // the first pass cleared the status words at the head of the workspace; the second pass reports
  // into the same words (the first failure wins)
  int* status = reinterpret_cast<int*>(w);
  rc = pl.use_pv_tc ? pv_tc_run(p, heads, pl.pv_tc, logits, w + pl.off_pass2, status, st)
                    : latent_pv_run(p, heads, pl.pv, logits, w + pl.off_pass2, status, st);
  if (rc != XKV_OK) return rc;
  const size_t off_partial = pl.use_pv_tc ? pl.pv_tc.off_partial : pl.pv.off_partial;
  const size_t off_lse = pl.use_pv_tc ? pl.pv_tc.off_lse : pl.pv.off_lse;
  const int pv_splits = pl.use_pv_tc ? pl.pv_tc.num_splits : pl.pv.num_splits;
  const float* partial = reinterpret_cast<const float*>(w + pl.off_pass2 + off_partial);
  const float* lse = reinterpret_cast<const float*>(w + pl.off_pass2 + off_lse);
  for (int i = 0; i < n; ++i) {
    const xkv_decode_params& li = layers[i];
    rc = launch_merge(partial, lse, li.out, p.dtype, p.batch, H, pv_splits, p.v_rank, li.value_dim, li.v_proj,
                      li.v_proj ? li.v_proj_heads : 1, li.vp_sb, li.vp_sh, li.vp_sr, li.vp_sd, li.o_sb, li.o_sh, st,
                      heads, i * H, li.lse_out, li.lse_sb);
    if (rc != XKV_OK) return rc;
  }
  return XKV_OK;
}

}  // namespace xkv
