/*
 * libxkv — C ABI of the B200 (sm_100a) decode-attention kernels.
 *
 * One decode step (q_len == 1) of grouped-query attention over a KV cache that is
 * dense, low-rank factorized (K = A.B, V = A_v.B_v) or an MLA latent, with optional
 * RoPE applied to the reconstructed keys.  Every entry point is asynchronous on the
 * CUDA stream passed in, allocates nothing on the device, keeps no pointer after it
 * returns, and reports failures as negative xkv_status codes (never aborts or traps).
 *
 * All tensors of one call share one element type (`dtype`); the innermost dimension of
 * every tensor is contiguous and the other dimensions are addressed by ELEMENT strides.
 * The caller owns inputs, outputs and the workspace (size from *_workspace_bytes()).
 *
 * The reference project is Python + Triton; each entry point names the reference
 * function(s) (path:line inside that project) whose device work it replaces.
 */
#ifndef XKV_H_
#define XKV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XKV_VERSION 1

#if defined(__GNUC__)
#define XKV_API __attribute__((visibility("default")))
#else
#define XKV_API
#endif

typedef enum xkv_status {
  XKV_OK = 0,
  XKV_ERR_BAD_ARG = -1,     /* null pointer, non-positive size, inconsistent shapes          */
  XKV_ERR_UNSUPPORTED = -2, /* valid request outside what the kernels cover (size limits)    */
  XKV_ERR_ALIGN = -3,       /* pointer / stride alignment the selected kernel needs          */
  XKV_ERR_WORKSPACE = -4,   /* workspace null or too small                                   */
  XKV_ERR_LAUNCH = -5,      /* CUDA reported an error at launch                              */
  XKV_ERR_TIMEOUT = -6,     /* a bounded device-side wait expired (read from the status word) */
  XKV_ERR_NO_DEVICE = -7,   /* no usable sm_100 device / driver entry point                  */
  XKV_ERR_SCRATCH_LIMIT = -8 /* xkv_decode_builtin_scratch(): request exceeds the built-in array */
} xkv_status;

typedef enum xkv_dtype { XKV_F32 = 0, XKV_BF16 = 1, XKV_F16 = 2 } xkv_dtype;

/* Where the attention logits come from. */
typedef enum xkv_score_mode {
  XKV_SCORE_DENSE = 0,      /* q[h] . K[b,l,kvh(h),:]                                        */
  XKV_SCORE_LATENT = 1,     /* (q[h] . k_proj^T) . A[b,l,:]  (+ q_tail[h] . k_tail[b,l,:])   */
  XKV_SCORE_RECON_ROPE = 2, /* q[h] . RoPE_l(A[b,l,:] . k_proj[b,kvh(h)])                    */
  XKV_SCORE_RECON = 3       /* q[h] . (A[b,l,:] . k_proj[b,kvh(h)])  (no rotation)           */
} xkv_score_mode;

/* Where the values come from. */
typedef enum xkv_value_mode {
  XKV_VALUE_DENSE = 0,      /* V[b,l,kvh(h),:]                                               */
  XKV_VALUE_LATENT = 1      /* (P . A_v[b,:,:]) . v_proj[head]; v_proj == NULL keeps latent  */
} xkv_value_mode;

#define XKV_FLAG_LOGITS_ONLY 1u  /* write sm_scale * logits to `logits`, skip softmax and P.V */
#define XKV_FLAG_FORCE_GENERIC 2u /* use the portable CUDA-core kernel even when a tensor-core
                                     kernel covers the shape (debugging / cross-checks)      */
#define XKV_FLAG_RECON_SINGLE_CTA 4u /* key reconstruction: keep one CTA per tile instead of CTA
                                     pairs that share each MMA (cross-checks)                */
#define XKV_FLAG_PV_MMA_SYNC 8u  /* two-pass decode: run the softmax + P.A_v pass on the mma.sync
                                     kernel instead of the tcgen05 one (cross-checks)         */
#define XKV_FLAG_LATENT_MMA_SYNC 32u /* shared-latent decode (MLA, absorbed caches): keep the mma.sync
                                     kernel where the tcgen05 CTA-pair kernel would run (cross-checks) */
#define XKV_FLAG_RECON_PAIR 16u  /* key reconstruction: ask for the CTA-pair variant where the
                                     library would not choose it by itself                    */

/*
 * One decode-attention call.  Shapes (H = num_heads, KVH = num_kv_heads, L = kv_len):
 *   q        (batch, H, head_dim)                       strides q_sb, q_sh
 *   q_tail   (batch, H, tail_dim)          or NULL      decoupled RoPE query part (MLA)
 *   k        DENSE : (batch, L, KVH, head_dim)          strides k_sb, k_sl, k_sh
 *            LATENT / RECON* : key latent A (batch, L, k_rank), strides k_sb, k_sl
 *   k_tail   (batch, L, tail_dim)          or NULL      decoupled RoPE key part (MLA)
 *   k_proj   (batch, k_proj_heads, k_rank, head_dim) addressed by kp_sb, kp_sh, kp_sr, kp_sd
 *            (B_k, or W_uk with swapped strides); k_proj_heads is KVH or H.  LATENT with
 *            k_proj == NULL means q is already in latent space (head_dim == k_rank).
 *   v        DENSE : (batch, L, KVH, value_dim)         strides v_sb, v_sl, v_sh
 *            LATENT: value latent A_v (batch, L, v_rank), strides v_sb, v_sl
 *   v_proj   (batch, v_proj_heads, v_rank, value_dim) by vp_sb, vp_sh, vp_sr, vp_sd, or NULL
 *   out      (batch, H, value_dim)   (value_dim == v_rank when v_proj == NULL)
 *   logits   (batch, H, L)           only with XKV_FLAG_LOGITS_ONLY
 * A batch stride of 0 broadcasts one matrix over the batch (shared B / W matrices).
 */
typedef struct xkv_decode_params {
  int32_t dtype;       /* xkv_dtype of every tensor                                         */
  int32_t score_mode;  /* xkv_score_mode                                                    */
  int32_t value_mode;  /* xkv_value_mode                                                    */
  uint32_t flags;
  int32_t batch, num_heads, num_kv_heads, kv_len;
  int32_t head_dim, value_dim, k_rank, v_rank, tail_dim;
  int32_t k_proj_heads, v_proj_heads;
  int32_t num_splits;  /* KV-split hint, 0 = choose from the SM count                        */
  int32_t pos_offset;  /* RoPE position of key row 0                                         */
  float sm_scale;      /* multiplies the logits                                              */
  float theta;         /* RoPE base, used when inv_freq == NULL                              */
  float logit_cap;     /* > 0: logits = cap * tanh(logits / cap)                             */
  const float* inv_freq; /* device, head_dim/2 floats, or NULL                               */
  const float* rope_table; /* device (kv_len, head_dim/2, 2) {cos, sin} for key rows 0..L-1, or
                              NULL to derive the angles from inv_freq / theta and pos_offset  */
  const void* q;      int64_t q_sb, q_sh;
  const void* q_tail; int64_t qt_sb, qt_sh;
  const void* k;      int64_t k_sb, k_sl, k_sh;
  const void* k_tail; int64_t kt_sb, kt_sl;
  const void* k_proj; int64_t kp_sb, kp_sh, kp_sr, kp_sd;
  const void* v;      int64_t v_sb, v_sl, v_sh;
  const void* v_proj; int64_t vp_sb, vp_sh, vp_sr, vp_sd;
  void* out;          int64_t o_sb, o_sh;
  void* logits;       int64_t lg_sb, lg_sh;
  const int32_t* kv_lens; /* device, `batch` entries, or NULL: row b attends to its first
                             min(kv_lens[b], kv_len) cache rows (ragged batches); 0 gives a zero row.
                             No counterpart in the reference, whose kernels take one length.       */
  float* lse_out;     int64_t lse_sb; /* optional (batch, H) fp32 at [b * lse_sb + h]: natural-log
                             sum-exp of the scaled logits of each head (-inf for an empty row).  With it the
                             results of calls over disjoint parts of a cache can be merged exactly
                             (xkv_merge), e.g. a factorized prefill cache plus a dense tail of fresh tokens:
                             flash_decoding/deepseek_mla/flash_decoding.py:66-255 in the reference.  NULL = off. */
  const void* mask;   int64_t mask_sb, mask_sh; /* optional additive mask of the call's dtype, added to
                             the scaled logits before the softmax: mask[b * mask_sb + h * mask_sh + token]; strides
                             of 0 broadcast over the batch / the heads (attention.py:60-64 in the reference).  Calls
                             with a mask run on the portable kernels.  NULL = no mask.                        */
} xkv_decode_params;

XKV_API int xkv_version(void);
/* sizeof(xkv_decode_params) as compiled into the library, for bindings to check their mirror. */
XKV_API size_t xkv_decode_params_size(void);
XKV_API const char* xkv_strerror(int status);

/* Name of the kernel family xkv_decode() would run for these parameters ("generic",
 * "recon_tc", ...), or NULL when they are rejected.  Host-only; launches nothing. */
XKV_API const char* xkv_decode_plan(const xkv_decode_params* p);

/* Bytes of device scratch xkv_decode() needs for these parameters (0 on bad parameters). */
XKV_API size_t xkv_decode_workspace_bytes(const xkv_decode_params* p);

/*
 * General entry point: any combination of score and value modes.  `stream` is a
 * cudaStream_t passed as void*.  Replaces the device work of every function below.
 */
XKV_API int xkv_decode(const xkv_decode_params* p, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Decode attention for callers that cannot allocate device memory.
 *
 * Some hosts of this library never get to call cudaMalloc: a plugin running inside a server
 * whose memory pool was sized and frozen at start-up, a real-time loop that must not touch the
 * allocator, a process whose device memory is entirely owned by another runtime.  For them this
 * entry point runs the same portable split-KV kernels as xkv_decode() (every score / value
 * mode and dtype) but takes its scratch from an array compiled into the library instead of a
 * caller workspace.  It calls no cudaMalloc / cudaFree and no allocating library routine; the
 * caller still passes inputs and outputs.  It has no counterpart in the reference, whose
 * wrappers allocate their intermediate buffers with torch on every call.
 *
 *  - The array is XKV_BUILTIN_SCRATCH_BYTES (8 MiB) of device memory on every GPU that loads
 *    the library, held until the process exits.  A request whose split-KV partials need more
 *    returns XKV_ERR_SCRATCH_LIMIT and launches nothing (lower num_splits or the batch, or use
 *    xkv_decode() with a workspace).  The tensor-core kernels are not used on this path.
 *  - The first call on each device resolves the array's device address (cudaGetSymbolAddress,
 *    with that device current) and keeps it for the life of the process.  Make that first call
 *    outside any stream capture.  The kept address does not survive a cudaDeviceReset of that
 *    device: a process that resets a device must not call this entry point on it afterwards.
 *  - All calls on one device share the one array, which keeps whatever the last call left in
 *    it; every call rewrites what it later reads, so stale contents are harmless, but two
 *    calls that overlap on the GPU (different streams, or concurrent host threads) race on
 *    it.  Serialise them.
 */
#define XKV_BUILTIN_SCRATCH_BYTES (8u << 20)
XKV_API int xkv_decode_builtin_scratch(const xkv_decode_params* p, void* stream);

/*
 * Synchronises `stream` and reads back the status words the last xkv_decode() on this workspace
 * left in its first 32 bytes: returns XKV_OK, or XKV_ERR_TIMEOUT when a bounded device-side
 * wait expired (detail[1..4], if detail != NULL, then hold role, tile, chunk and step of the
 * first wait that gave up), or XKV_ERR_LAUNCH when CUDA reports an error.  detail has 8 entries.
 * No counterpart in the reference (its kernels have no device-side waits).
 */
XKV_API int xkv_workspace_status(const void* workspace, void* stream, int32_t* detail);

/*
 * Named entry points.  Each checks that the parameter block describes its operation and
 * then runs xkv_decode(); they exist so that a binding reads like the reference call.
 *
 * xkv_dense_decode       dense K and V.  Replaces attention.py:7-90 (group_query_attention),
 *                        attention.py:184-191 (group_query_attention_fa) and
 *                        flash_decoding/gqa.py:339-434 (decode_attention_fwd).
 * xkv_absorbed_decode    factorized K and/or V without RoPE (absorbed form).  Replaces
 *                        attention.py:202-274 (_factorized_v_only), attention.py:276-357
 *                        (_factorized) and flash_recontruction/fused_attention/no_pe/
 *                        v1.py:365-474, v2.py:364-474, v1_k_only.py:368-465.
 * xkv_recon_rope_decode  K tile rebuilt as A.B, rotated, dotted with q, softmax, P.V in one
 *                        pass.  Replaces attention.py:360-431 (_factorized_RoPE) including its
 *                        call into flash_recontruction/qAB/v1.py:90-148.
 * xkv_qab_logits         logits only, with or without RoPE.  Replaces
 *                        flash_recontruction/qAB/v1.py:90-148, v2.py:132-187, v3.py:84-142,
 *                        v4.py:85-143 and qAB_no_pe/v1.py:78-135, v2.py:72-130.
 * xkv_mla_decode         latent attention with a decoupled RoPE key; optional W_uk / W_uv
 *                        absorption.  Replaces flash_decoding/mla2/mla_flash_decoding.py:6-62
 *                        and :66-130, and flash_decoding/mla.py:388-440.
 */
XKV_API int xkv_dense_decode(const xkv_decode_params* p, void* ws, size_t ws_bytes, void* stream);
XKV_API int xkv_absorbed_decode(const xkv_decode_params* p, void* ws, size_t ws_bytes, void* stream);
XKV_API int xkv_recon_rope_decode(const xkv_decode_params* p, void* ws, size_t ws_bytes, void* stream);
XKV_API int xkv_qab_logits(const xkv_decode_params* p, void* ws, size_t ws_bytes, void* stream);
XKV_API int xkv_mla_decode(const xkv_decode_params* p, void* ws, size_t ws_bytes, void* stream);

/*
 * Cross-layer group decode: `num_layers` consecutive layers share the key latent (and the
 * value latent when values are factorized); each layer has its own q, k_proj, v_proj (and
 * dense V) and its own output.  layers[i] is a full parameter block; the blocks must agree on
 * every size and on the shared latent pointers.  No single reference function does this: per
 * layer it is attention.py:360-431 / :202-274; the sharing is the xKV cross-layer scheme.
 */
XKV_API size_t xkv_group_decode_workspace_bytes(const xkv_decode_params* layers, int num_layers);
XKV_API int xkv_group_decode(const xkv_decode_params* layers, int num_layers, void* ws, size_t ws_bytes,
                     void* stream);

/*
 * LSE-weighted merge of split-KV partial results, exposed for callers that keep their own
 * partials.  partial_o (batch, H, num_splits, dim) fp32 normalised per split, lse
 * (batch, H, num_splits) fp32 (-inf marks an empty split), out (batch, H, dim) of `dtype`.
 * Replaces flash_decoding/gqa.py:241-299 (stage 2) and mla2/stage2.py:41-99.
 */
XKV_API int xkv_merge(const float* partial_o, const float* lse, void* out, int dtype, int batch,
              int num_heads, int num_splits, int dim, int64_t o_sb, int64_t o_sh, void* stream);

/* Fill cos_sin[(l * half + j) * 2 + {0,1}] = {cos, sin}(float(pos_offset + l) * inv_freq[j]),
 * the table the RoPE kernels read.  inv_freq may be NULL (computed from theta, dim = 2*half).
 * Replaces flash_recontruction/rope/sin_cos.py:72-99 (rotary_sin_cos). */
XKV_API int xkv_rope_table(float* cos_sin, int kv_len, int half, int pos_offset, float theta,
                   const float* inv_freq, void* stream);

/*
 * Rotate the decode-step queries to their positions: out[b, h, :] = RoPE(q[b, h, :], pos_b) in the
 * half-split form (pairs j, j + head_dim/2), angle = float(pos_b) * inv_freq[j].  pos_b is
 * positions[b] (device int32, one per batch row) when positions != NULL, else `position`.  q and out
 * are (batch, num_heads, head_dim) of `dtype` with element strides; out may alias q.  inv_freq may be
 * NULL (derived from theta).  Replaces the rotation the caller of the reference's kernels does itself
 * with flash_recontruction/rope/rope_ref.py:11-21 (the kernels use q as given, qAB/v1.py:71-77).
 */
XKV_API int xkv_rope_query(const void* q, void* out, int dtype, int batch, int num_heads, int head_dim,
                   int64_t q_sb, int64_t q_sh, int64_t o_sb, int64_t o_sh, int position,
                   const int32_t* positions, float theta, const float* inv_freq, void* stream);

/*
 * Append one token per sequence to a factorized cache: latent[b, pos_b, :] = x[b, :] . proj, with x
 * (batch, in_dim) the new key (or value) row of all KV heads side by side, proj (in_dim, rank) the
 * map into latent space (the pseudo-inverse of the cache's B matrix) addressed as
 * proj[c * p_sc + r * p_sr], and latent (batch, capacity, rank) the cache's A.  pos_b as in
 * xkv_rope_query; rows whose position is outside [0, capacity) are left alone.  fp32 accumulation.
 * The reference has no counterpart: its caches are synthetic and never grow
 * (flash_decoding/gqa.py:60,89 take one constant length).
 */
XKV_API int xkv_latent_append(const void* x, int64_t x_sb, const void* proj, int64_t p_sc, int64_t p_sr,
                      void* latent, int64_t l_sb, int64_t l_sl, const int32_t* positions, int position,
                      int dtype, int batch, int in_dim, int rank, int capacity, void* stream);

/*
 * All-gather of per-rank output shards with plain peer stores over NVLink (no collective library), for
 * steps short enough that a collective's latency shows.  bufs[r] (r < world) is rank r's gather buffer as
 * mapped in THIS process (symmetric / peer-mapped memory of one layout: 2 halves x world slots x
 * shard_bytes, then 256 bytes at flags_offset, zero before the first call: `world` uint32 flag words and, from
 * byte 128, the kernel's own arrival counters).  The launch copies
 * `local` into slot `rank` of half (epoch & 1) of every rank's buffer, publishes `epoch` in every rank's
 * flag word `rank`, and returns (on the stream) once this rank's own flag words all show `epoch`: its
 * half then holds every rank's shard.  `epoch` must grow by one per call on every rank, starting at 1.  A
 * peer that does not show up within a second leaves XKV_ERR_TIMEOUT in status_dev[0] (role 40, peer,
 * epoch in [1..3]) instead of hanging.  The reference has no multi-GPU code; this replaces the
 * all_gather_into_tensor the batch-sharded decode ends with.
 */
XKV_API int xkv_peer_allgather(const void* local, size_t shard_bytes, void* const* bufs, size_t flags_offset, int rank,
                       int world, uint32_t epoch, int* status_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* XKV_H_ */
