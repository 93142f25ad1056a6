// C ABI of libxkv: parameter validation, kernel selection, named entry points.
#include "xkv_internal.h"
#include <string.h>

namespace xkv {
namespace {

bool is_recon(int m) { return m == XKV_SCORE_RECON || m == XKV_SCORE_RECON_ROPE; }

int validate(const xkv_decode_params* p) {
  if (!p) return XKV_ERR_BAD_ARG;
  if (p->dtype < XKV_F32 || p->dtype > XKV_F16) return XKV_ERR_BAD_ARG;
  if (p->score_mode < XKV_SCORE_DENSE || p->score_mode > XKV_SCORE_RECON) return XKV_ERR_BAD_ARG;
  if (p->value_mode < XKV_VALUE_DENSE || p->value_mode > XKV_VALUE_LATENT) return XKV_ERR_BAD_ARG;
  if (p->batch <= 0 || p->num_heads <= 0 || p->num_kv_heads <= 0 || p->kv_len <= 0) return XKV_ERR_BAD_ARG;
  if (p->head_dim <= 0) return XKV_ERR_BAD_ARG;
  if (p->num_heads % p->num_kv_heads != 0) return XKV_ERR_BAD_ARG;
  if (p->num_splits < 0) return XKV_ERR_BAD_ARG;
  if (!p->q || !p->k) return XKV_ERR_BAD_ARG;
  const bool logits_only = (p->flags & XKV_FLAG_LOGITS_ONLY) != 0;
  if (p->tail_dim < 0) return XKV_ERR_BAD_ARG;
  if (p->tail_dim > 0) {
    if (p->score_mode != XKV_SCORE_LATENT) return XKV_ERR_BAD_ARG;
    if (!p->q_tail || !p->k_tail) return XKV_ERR_BAD_ARG;
  }
  if (p->score_mode != XKV_SCORE_DENSE) {
    if (p->k_rank <= 0) return XKV_ERR_BAD_ARG;
    if (is_recon(p->score_mode) && !p->k_proj) return XKV_ERR_BAD_ARG;
    if (p->k_proj) {
      if (p->k_proj_heads <= 0 || p->num_heads % p->k_proj_heads != 0) return XKV_ERR_BAD_ARG;
      if (is_recon(p->score_mode) && p->k_proj_heads != p->num_kv_heads) return XKV_ERR_BAD_ARG;
    } else if (p->head_dim != p->k_rank) {
      return XKV_ERR_BAD_ARG;
    }
    if (p->score_mode == XKV_SCORE_RECON_ROPE && (p->head_dim & 1)) return XKV_ERR_BAD_ARG;
  }
  if (logits_only) {
    if (!p->logits) return XKV_ERR_BAD_ARG;
  } else {
    if (!p->v || !p->out || p->value_dim <= 0) return XKV_ERR_BAD_ARG;
    if (p->value_mode == XKV_VALUE_LATENT) {
      if (p->v_rank <= 0) return XKV_ERR_BAD_ARG;
      if (p->v_proj) {
        if (p->v_proj_heads <= 0 || p->num_heads % p->v_proj_heads != 0) return XKV_ERR_BAD_ARG;
      } else if (p->value_dim != p->v_rank) {
        return XKV_ERR_BAD_ARG;
      }
    }
  }
  return XKV_OK;
}

enum class Path { kNone, kGeneric, kReconTc, kDenseTc, kLatentTc, kLatentPair, kTwoPass };

struct Plans {
  xkv_decode_params rewritten;   // the call as the chosen kernel sees it (see as_latent)
  GenericPlan generic;
  ReconTcPlan recon;
  DenseTcPlan dense;
  LatentTcPlan latent;
  TwoPassPlan two_pass;
};

// A dense cache with ONE KV head (the packed MLA layout: keys [latent | rope], values a prefix of the
// keys or a separate buffer) is a shared-latent call whose query is already in latent space.
bool as_latent(const xkv_decode_params& p, xkv_decode_params* t) {
  if (p.score_mode != XKV_SCORE_DENSE || p.value_mode != XKV_VALUE_DENSE || p.num_kv_heads != 1) return false;
  if (p.flags & XKV_FLAG_LOGITS_ONLY) return false;
  *t = p;
  t->score_mode = XKV_SCORE_LATENT;
  t->value_mode = XKV_VALUE_LATENT;
  t->k_rank = p.head_dim;
  t->k_proj = nullptr;
  t->v_rank = p.value_dim;
  t->v_proj = nullptr;
  t->tail_dim = 0;
  return true;
}

Path select(const xkv_decode_params& p, Plans* pl) {
  GenericPlan* gp = &pl->generic;
  pl->rewritten = p;
  if (!(p.flags & XKV_FLAG_FORCE_GENERIC)) {
    if (recon_tc_supported(p) && recon_tc_plan(p, &pl->recon)) return Path::kReconTc;
    if (dense_tc_supported(p) && dense_tc_plan(p, &pl->dense)) return Path::kDenseTc;
    if (latent_pair_supported(p) && latent_pair_plan(p, &pl->latent)) return Path::kLatentPair;
    if (latent_tc_supported(p) && latent_tc_plan(p, &pl->latent)) return Path::kLatentTc;
    xkv_decode_params t;
    if (as_latent(p, &t)) {
      pl->rewritten = t;
      if (latent_pair_supported(t) && latent_pair_plan(t, &pl->latent)) return Path::kLatentPair;
      if (latent_tc_supported(t) && latent_tc_plan(t, &pl->latent)) return Path::kLatentTc;
      pl->rewritten = p;
    }
    if (two_pass_supported(&p, 1) && two_pass_plan(&p, 1, &pl->two_pass)) return Path::kTwoPass;
  }
  if (generic_plan(p, gp)) return Path::kGeneric;
  return Path::kNone;
}

int check_mode(const xkv_decode_params* p, bool ok) {
  if (!p) return XKV_ERR_BAD_ARG;
  return ok ? XKV_OK : XKV_ERR_BAD_ARG;
}

}  // namespace
}  // namespace xkv

using namespace xkv;

extern "C" {

int xkv_version(void) { return XKV_VERSION; }

size_t xkv_decode_params_size(void) { return sizeof(xkv_decode_params); }

const char* xkv_strerror(int status) {
  switch (status) {
    case XKV_OK: return "ok";
    case XKV_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size or inconsistent shapes)";
    case XKV_ERR_UNSUPPORTED: return "shape outside the limits of the kernels";
    case XKV_ERR_ALIGN: return "pointer or stride not aligned as the kernel requires";
    case XKV_ERR_WORKSPACE: return "workspace missing or too small";
    case XKV_ERR_LAUNCH: return "CUDA launch failed";
    case XKV_ERR_TIMEOUT: return "bounded device-side wait expired";
    case XKV_ERR_NO_DEVICE: return "no usable sm_100 device or driver entry point";
    case XKV_ERR_SCRATCH_LIMIT:
      return "request needs more scratch than the library's built-in array holds; use xkv_decode() with a workspace";
    default: return "unknown status";
  }
}

const char* xkv_decode_plan(const xkv_decode_params* p) {
  if (validate(p) != XKV_OK) return nullptr;
  Plans pl;
  switch (select(*p, &pl)) {
    case Path::kReconTc: return "recon_tc";
    case Path::kDenseTc: return "dense_tc";
    case Path::kLatentTc: return "latent_tc";
    case Path::kLatentPair: return "latent_pair";
    case Path::kTwoPass: return "two_pass";
    case Path::kGeneric: return "generic";
    default: return nullptr;
  }
}

size_t xkv_decode_workspace_bytes(const xkv_decode_params* p) {
  if (validate(p) != XKV_OK) return 0;
  Plans pl;
  switch (select(*p, &pl)) {
    case Path::kReconTc: return pl.recon.total_bytes;
    case Path::kDenseTc: return pl.dense.total_bytes;
    case Path::kLatentTc: return pl.latent.total_bytes;
    case Path::kLatentPair: return pl.latent.total_bytes;
    case Path::kTwoPass: return pl.two_pass.total_bytes;
    case Path::kGeneric: return pl.generic.total_bytes;
    default: return 0;
  }
}

int xkv_decode(const xkv_decode_params* p, void* ws, size_t ws_bytes, void* stream) {
  int rc = validate(p);
  if (rc != XKV_OK) return rc;
  Plans pl;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (select(*p, &pl)) {
    case Path::kReconTc:
      if (!ws || ws_bytes < pl.recon.total_bytes) return XKV_ERR_WORKSPACE;
      return recon_tc_decode(*p, pl.recon, ws, st);
    case Path::kDenseTc:
      if (!ws || ws_bytes < pl.dense.total_bytes) return XKV_ERR_WORKSPACE;
      return dense_tc_decode(*p, pl.dense, ws, st);
    case Path::kLatentTc:
      if (!ws || ws_bytes < pl.latent.total_bytes) return XKV_ERR_WORKSPACE;
      return latent_tc_decode(pl.rewritten, pl.latent, ws, st);
    case Path::kLatentPair:
      if (!ws || ws_bytes < pl.latent.total_bytes) return XKV_ERR_WORKSPACE;
      return latent_pair_decode(pl.rewritten, pl.latent, ws, st);
    case Path::kTwoPass:
      if (!ws || ws_bytes < pl.two_pass.total_bytes) return XKV_ERR_WORKSPACE;
      return two_pass_decode(p, 1, pl.two_pass, ws, st);
    case Path::kGeneric:
      if (!ws || ws_bytes < pl.generic.total_bytes) return XKV_ERR_WORKSPACE;
      return generic_decode(*p, pl.generic, ws, st);
    default:
      return XKV_ERR_UNSUPPORTED;
  }
}

int xkv_decode_builtin_scratch(const xkv_decode_params* p, void* stream) {
  int rc = validate(p);
  if (rc != XKV_OK) return rc;
  GenericPlan gp;
  if (!generic_plan(*p, &gp)) return XKV_ERR_UNSUPPORTED;
  return generic_decode_builtin_scratch(*p, gp, static_cast<cudaStream_t>(stream));
}

int xkv_dense_decode(const xkv_decode_params* p, void* ws, size_t n, void* st) {
  int rc = check_mode(p, p && p->score_mode == XKV_SCORE_DENSE && p->value_mode == XKV_VALUE_DENSE &&
                             !(p->flags & XKV_FLAG_LOGITS_ONLY));
  return rc != XKV_OK ? rc : xkv_decode(p, ws, n, st);
}

int xkv_absorbed_decode(const xkv_decode_params* p, void* ws, size_t n, void* st) {
  int rc = check_mode(p, p && !(p->flags & XKV_FLAG_LOGITS_ONLY) && p->tail_dim == 0 &&
                             (p->score_mode == XKV_SCORE_LATENT || p->score_mode == XKV_SCORE_DENSE) &&
                             (p->score_mode == XKV_SCORE_LATENT || p->value_mode == XKV_VALUE_LATENT));
  return rc != XKV_OK ? rc : xkv_decode(p, ws, n, st);
}

int xkv_recon_rope_decode(const xkv_decode_params* p, void* ws, size_t n, void* st) {
  int rc = check_mode(p, p && p->score_mode == XKV_SCORE_RECON_ROPE && !(p->flags & XKV_FLAG_LOGITS_ONLY));
  return rc != XKV_OK ? rc : xkv_decode(p, ws, n, st);
}

int xkv_qab_logits(const xkv_decode_params* p, void* ws, size_t n, void* st) {
  int rc = check_mode(p, p && (p->flags & XKV_FLAG_LOGITS_ONLY) && p->score_mode != XKV_SCORE_DENSE);
  return rc != XKV_OK ? rc : xkv_decode(p, ws, n, st);
}

int xkv_mla_decode(const xkv_decode_params* p, void* ws, size_t n, void* st) {
  int rc = check_mode(p, p && p->score_mode == XKV_SCORE_LATENT && p->value_mode == XKV_VALUE_LATENT &&
                             p->num_kv_heads == 1 && !(p->flags & XKV_FLAG_LOGITS_ONLY));
  return rc != XKV_OK ? rc : xkv_decode(p, ws, n, st);
}

// Group decode: the layers share the key latent.  Groups the tensor-core kernel covers run as ONE
// launch whose CTAs for the different layers of a (split, batch row) are scheduled together, so a
// latent tile is fetched from HBM once and served from L2 to the other layers.  Anything else
// runs layer by layer on the shared workspace.
static int group_check(const xkv_decode_params* layers, int n) {
  if (!layers || n <= 0) return XKV_ERR_BAD_ARG;
  for (int i = 0; i < n; ++i) {
    int rc = validate(&layers[i]);
    if (rc != XKV_OK) return rc;
    const xkv_decode_params &a = layers[0], &b = layers[i];
    if (a.dtype != b.dtype || a.score_mode != b.score_mode || a.value_mode != b.value_mode ||
        a.batch != b.batch || a.num_heads != b.num_heads || a.num_kv_heads != b.num_kv_heads ||
        a.kv_len != b.kv_len || a.head_dim != b.head_dim || a.value_dim != b.value_dim ||
        a.k_rank != b.k_rank || a.v_rank != b.v_rank || a.tail_dim != b.tail_dim)
      return XKV_ERR_BAD_ARG;
    if (a.score_mode != XKV_SCORE_DENSE && a.k != b.k) return XKV_ERR_BAD_ARG;
    if (a.value_mode == XKV_VALUE_LATENT && a.v != b.v) return XKV_ERR_BAD_ARG;
  }
  return XKV_OK;
}

size_t xkv_group_decode_workspace_bytes(const xkv_decode_params* layers, int n) {
  if (group_check(layers, n) != XKV_OK) return 0;
  ReconTcPlan rp;
  if (recon_tc_group_supported(layers, n) && recon_tc_group_plan(layers, n, &rp)) return rp.total_bytes;
  TwoPassPlan tp;
  if (two_pass_supported(layers, n) && two_pass_plan(layers, n, &tp)) return tp.total_bytes;
  size_t mx = 0;
  for (int i = 0; i < n; ++i) {
    size_t b = xkv_decode_workspace_bytes(&layers[i]);
    if (b == 0) return 0;
    if (b > mx) mx = b;
  }
  return mx;
}

int xkv_group_decode(const xkv_decode_params* layers, int n, void* ws, size_t ws_bytes, void* stream) {
  int rc = group_check(layers, n);
  if (rc != XKV_OK) return rc;
  ReconTcPlan rp;
  if (recon_tc_group_supported(layers, n) && recon_tc_group_plan(layers, n, &rp)) {
    if (!ws || ws_bytes < rp.total_bytes) return XKV_ERR_WORKSPACE;
    return recon_tc_group_decode(layers, n, rp, ws, static_cast<cudaStream_t>(stream), nullptr);
  }
  TwoPassPlan tp;
  if (two_pass_supported(layers, n) && two_pass_plan(layers, n, &tp)) {
    if (!ws || ws_bytes < tp.total_bytes) return XKV_ERR_WORKSPACE;
    return two_pass_decode(layers, n, tp, ws, static_cast<cudaStream_t>(stream));
  }
  for (int i = 0; i < n; ++i) {
    rc = xkv_decode(&layers[i], ws, ws_bytes, stream);
    if (rc != XKV_OK) return rc;
  }
  return XKV_OK;
}

int xkv_workspace_status(const void* workspace, void* stream, int32_t* detail) {
  if (!workspace) return XKV_ERR_BAD_ARG;
  int32_t host[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess) return XKV_ERR_LAUNCH;
  if (cudaMemcpy(host, workspace, sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess) return XKV_ERR_LAUNCH;
  if (detail) memcpy(detail, host, sizeof(host));
  return host[0] > 0 ? XKV_ERR_LAUNCH : host[0];
}

int xkv_merge(const float* partial_o, const float* lse, void* out, int dtype, int batch, int num_heads,
              int num_splits, int dim, int64_t o_sb, int64_t o_sh, void* stream) {
  if (!partial_o || !lse || !out || batch <= 0 || num_heads <= 0 || num_splits <= 0 || dim <= 0)
    return XKV_ERR_BAD_ARG;
  return launch_merge(partial_o, lse, out, dtype, batch, num_heads, num_splits, dim, dim, nullptr, 1, 0, 0,
                      0, 0, o_sb, o_sh, static_cast<cudaStream_t>(stream));
}

int xkv_rope_table(float* cos_sin, int kv_len, int half, int pos_offset, float theta,
                   const float* inv_freq, void* stream) {
  if (!cos_sin || kv_len <= 0 || half <= 0) return XKV_ERR_BAD_ARG;
  return launch_rope_table(cos_sin, kv_len, half, pos_offset, theta, inv_freq,
                           static_cast<cudaStream_t>(stream));
}

int xkv_rope_query(const void* q, void* out, int dtype, int batch, int num_heads, int head_dim, int64_t q_sb,
                   int64_t q_sh, int64_t o_sb, int64_t o_sh, int position, const int32_t* positions, float theta,
                   const float* inv_freq, void* stream) {
  if (!q || !out || batch <= 0 || num_heads <= 0 || head_dim <= 0 || (head_dim & 1)) return XKV_ERR_BAD_ARG;
  if (!inv_freq && !(theta > 0.f)) return XKV_ERR_BAD_ARG;
  return launch_rope_query(q, out, dtype, batch, num_heads, head_dim, q_sb, q_sh, o_sb, o_sh, position, positions,
                           theta, inv_freq, static_cast<cudaStream_t>(stream));
}

int xkv_latent_append(const void* x, int64_t x_sb, const void* proj, int64_t p_sc, int64_t p_sr, void* latent,
                      int64_t l_sb, int64_t l_sl, const int32_t* positions, int position, int dtype, int batch,
                      int in_dim, int rank, int capacity, void* stream) {
  if (!x || !proj || !latent || batch <= 0 || in_dim <= 0 || rank <= 0 || capacity <= 0) return XKV_ERR_BAD_ARG;
  return launch_latent_append(x, x_sb, proj, p_sc, p_sr, latent, l_sb, l_sl, positions, position, dtype, batch,
                              in_dim, rank, capacity, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
