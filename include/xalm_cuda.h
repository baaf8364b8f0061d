/* =============================================================================================
 * xalm_cuda.h — C ABI of the B200 (sm_100a) `-d cuda` backend for Xalm's transformer forward pass.
 *
 * The reference has no plugin/FFI interface; its only device seam is three C++ call sites
 * (SURVEY.md §8b).  Each entry point below names the reference interface it stands in for.
 * Paths are relative to the reference tree (jubruckne/Xalm).
 *
 *   - nothing but POD, raw pointers and sizes crosses this boundary; no exceptions: every call
 *     returns 0 on success or a non-zero xalm_status, and xalm_cuda_last_error() describes it;
 *   - the backend owns all device memory (weights, KV cache, scratch) behind the opaque handle;
 *   - there is NO CPU fallback: without a usable CUDA device every compute call fails.
 * ============================================================================================= */
#ifndef XALM_CUDA_H
#define XALM_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XALM_CUDA_ABI_VERSION 1

/* Tensor element types.  0..9: `Type` ids, src/types.h:505-514.  1007..1012: the gguf-style block
 * formats convert.py writes (XType values, convert.py:56-61; layouts quants.py:281-464,638-683) which
 * the reference runtime never learned to load.  2007: convert.py's qi8 (:538-551). */
enum xalm_type {
	XALM_UNKNOWN = 0,
	XALM_F32 = 1, XALM_F16 = 2, XALM_BF16 = 3,
	XALM_F8_E2M5 = 4, XALM_F8_E3M4 = 5, XALM_F8_E4M3 = 6, XALM_F8_E5M2 = 7,
	XALM_U8 = 8, XALM_Q8 = 9,
	XALM_Q4_0 = 1007, XALM_Q4_1 = 1008, XALM_Q5_0 = 1009, XALM_Q5_1 = 1010, XALM_Q8_0 = 1011, XALM_TQ1_0 = 1012,
	XALM_QI8 = 2007
};

/* InferenceMode, src/model.h:249-252 */
enum xalm_mode { XALM_HYDRATE_KV_CACHE = 0, XALM_OUTPUT_LOGITS = 1 };
/* ActivationType, src/model.h:12-15 */
enum xalm_act { XALM_GELU = 0, XALM_SILU = 1 };

enum xalm_status {
	XALM_OK = 0,
	XALM_ERR_INVALID = 1,      /* bad argument / shape / unknown tensor name (load-time std::invalid_argument in the reference) */
	XALM_ERR_UNSUPPORTED = 2,  /* dtype the op does not take (infer.cpp:211-214, :248-249) */
	XALM_ERR_CUDA = 3,         /* CUDA runtime / driver error, or no device */
	XALM_ERR_STATE = 4,        /* call out of order (forward before finalize, missing tensors, ...) */
	XALM_ERR_COMM = 5          /* NCCL error */
};

/* Config, src/model.h:25-42 (same fields, same order; enums as int). */
typedef struct xalm_config {
	int dim;
	int hidden_dim;
	int head_dim;
	int n_layers;
	int n_heads;
	int n_kv_heads;
	int vocab_size;
	int max_seq_len;      /* after the 4096 clamp / -T override of Config::from_xalm (model.h:54-59) */
	float rope_theta;
	int rotary_dim;
	float norm_eps;
	int act;              /* xalm_act */
	int norm_type;        /* 0 = RMSNorm (the only LayerNormType, model.h:17-19) */
	float qkv_clip;       /* FLT_MAX when the checkpoint has none (model.h:84-85) */
	int tie_word_embeddings;
} xalm_config;

typedef struct xalm_cuda_model xalm_cuda_model; /* opaque: Model + InferenceState + KV caches on one GPU */

/* ---- diagnostics ------------------------------------------------------------------------- */
int xalm_cuda_abi_version(void);
/* Message for the last failing call on this thread ("" if none). Stands in for the reference's exceptions. */
const char* xalm_cuda_last_error(void);
int xalm_cuda_device_count(int* count);
/* (block elements, block bytes) of a type — Type::bit_size (types.h:350) generalised to quants.py:45-77. */
int xalm_cuda_type_info(int type_id, int* block_elems, int* block_bytes);

/* ---- model lifecycle: Model::from_xalm (model.cpp:48-118) + the commented-out
 *      `model.cuda(); state.cuda();` (main.cpp:211-212, :283-284) ------------------------------ */
/* tp_rank/tp_size: tensor-parallel shard this handle holds (1 GPU: 0/1).  Sharding per SURVEY.md §8e. */
int xalm_cuda_create(const xalm_config* cfg, int device, int tp_rank, int tp_size, xalm_cuda_model** out);
/* One call per tensor of model.cpp:83-114 ("embed.weight", "l.{i}.attn.{norm,q,k,v,down}.weight",
 * "l.{i}.mlp.{norm,gate,down,up}.weight", "output.norm.weight", "output.weight").  `shape` is the ELEMENT
 * shape (rows, cols), `data` the full (unsharded) host tensor in its on-disk byte layout; the backend keeps
 * only this rank's shard.  The host buffer may be freed on return. */
int xalm_cuda_upload_tensor(xalm_cuda_model* m, const char* name, int type_id, const int* shape, int rank,
                            const void* data, size_t nbytes);
/* Shard-aware upload for tensor-parallel handles, so that a rank reads / generates only what it keeps (the reference loader it
 * stands in for reads every tensor whole, model.cpp:48-118).  xalm_cuda_shard_range: range4 = {row0, row1, col0, col1} of the
 * ELEMENT shape this rank keeps of tensor `name` (norms and the embedding table: everything).  xalm_cuda_upload_tensor_shard:
 * `data` holds exactly that block, dense, in on-disk bytes (rows of (col1 - col0) elements); `shape` is still the full shape. */
int xalm_cuda_shard_range(xalm_cuda_model* m, const char* name, int* range4);
int xalm_cuda_upload_tensor_shard(xalm_cuda_model* m, const char* name, int type_id, const int* shape, int rank, const int* range4,
                                  const void* data, size_t nbytes);
/* Page-locked host memory for upload staging (H2D copies from it run at full PCIe rate and may be asynchronous). */
void* xalm_cuda_host_alloc(size_t nbytes);
void xalm_cuda_host_free(void* p);
/* Checks every tensor arrived, builds fused/concatenated device layouts, captures the per-token CUDA graphs. */
int xalm_cuda_finalize(xalm_cuda_model* m);
void xalm_cuda_destroy(xalm_cuda_model* m);

/* ---- model families described by a config.json -------------------------------------------------------------------------
 * The handle-based calls of this header serve every model family; a handle knows its family.  Llama/Mistral checkpoints
 * (.xalm) are created with xalm_cuda_create above.  A model folder with a config.json ("architecture": "<name>") and a
 * model.safetensors is created here: the backend parses the JSON text itself and picks the family registered under that
 * name (XALM_ERR_UNSUPPORTED when this build carries none).  Then, as for every family: xalm_cuda_upload_tensor once per
 * tensor (names as in the safetensors header; XALM_BF16 / XALM_F16 / XALM_F32 payloads), xalm_cuda_finalize,
 * xalm_cuda_prefill / xalm_cuda_forward for the running sequence, xalm_cuda_release when it ends.
 *   max_tokens: the most positions a sequence may hold (sizes the cache; windowed layers keep a ring of their window only).
 *   precision:  XALM_PRECISION_BF16 = the serving mode (16-bit matrix operands and K/V cache, fp32 accumulation, fp32 for
 *               norms, scores, softmax, recurrent state and the residual stream);
 *               XALM_PRECISION_F32  = everything in IEEE fp32 (no TF32), the K/V cache included. */
enum xalm_precision { XALM_PRECISION_BF16 = 0, XALM_PRECISION_F32 = 1 };
int xalm_cuda_create_json(const char* config_json, int device, int max_tokens, int precision, xalm_cuda_model** out);
/* Model families linked into this build ("Llama", "Nabalix", "Bolovik", ...). */
int xalm_cuda_family_count(void);
const char* xalm_cuda_family_name(int index);
/* The sequence is over: what it holds in the K/V cache and the recurrent state is given back; the next call starts at
 * position 0.  (Llama handles: a no-op, their ring is overwritten by position.) */
int xalm_cuda_release(xalm_cuda_model* m);
/* For loaders: tensor `index` the model expects (name, element shape of `*rank` <= 4 dims); XALM_ERR_INVALID past the last. */
int xalm_cuda_expected_tensor(xalm_cuda_model* m, int index, char* name, size_t name_cap, int* shape4, int* rank);
/* Integer properties by name: "vocab_size", "dim", "n_layers", "max_tokens", "position" (tokens the sequence holds). */
int xalm_cuda_model_info(xalm_cuda_model* m, const char* key, long long* value);

/* ---- mechanism ops: the sequence-mixing kernels of the config.json families, one call each (host arrays in and out, fp32) -----
 * They launch the kernels the families run, so a test holds each mechanism against a plain restatement.
 *
 * swa_attention: softmax attention over a sliding window (position i sees j with 0 <= i - j < window) for the T positions
 *   pos0 .. pos0+T-1.  q (T, H*d); k (pos0+T, G*d) and v (pos0+T, G*dv) hold EVERY position from 0 — the call lays them into a
 *   ring of `ring` slots (slot = position mod ring) as the cache manager would, so positions older than the ring are gone.
 *   score = scale q.k -> softcap * tanh(./softcap) (softcap 0: none) -> minus r1[h] * log1p(r2[h] (i - j)) (r1/r2 NULL: none) ->
 *   mixed across heads by talk (H, H) (NULL: none) -> softmax -> times v -> times sigmoid(gate (T, H*dv)) (NULL: none).
 *   n_splits > 1 splits the keys over CTAs as one-token steps do; cache_bf16 stores the ring in bf16.
 * hgrn2: S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T, o_t = S_t^T q_t per head, q = silu(qz), f = lower + (1 - lower) sigmoid(fz + f_bias)
 *   (f_bias / lower NULL: 0), o RMS-normed over dv with norm_w (NULL: no norm).  qz, fz (T, H*d); v (T, H*dv); state (H, d, dv) is
 *   read and written; out (T, H*dv).
 * hyper_norm: h[t] = rmsnorm(sum_s a[s] xs[s][t]) * (one_plus ? 1 + w : w); xs (S, T, W); a NULL: every coefficient 1.
 * dual_norm_hyper: y = 1/2 (rmsnorm(a) wa + rmsnorm(b) wb); xs[t'] <- sum_s mix[s, t'] xs[s] + out_coef[t'] * scale * y, all streams
 *   from the old ones (mix NULL: identity; out_coef NULL: ones; scale NULL: none).  xs (S, T, W) is read and written.
 * glu_rows: out (T, ff) = g * sigmoid(alpha g) * (u + 1), g = min(x Wg^T, limit), u = clamp(x Wu^T, -limit, limit); w_bf16 rounds the
 *   weights to bf16 first (the serving layout). */
int xalm_cuda_swa_attention(float* out, const float* q, const float* gate, const float* k, const float* v, int T, int pos0, int H, int G, int d, int dv,
                            int window, float scale, float softcap, const float* r1, const float* r2, const float* talk, int ring, int n_splits,
                            int cache_bf16);
int xalm_cuda_hgrn2(float* out, float* state, const float* qz, const float* fz, const float* v, int T, int H, int d, int dv, const float* f_bias,
                    const float* lower, const float* norm_w, float eps);
int xalm_cuda_hyper_norm(float* h, const float* xs, int S, int T, int W, const float* a, const float* w, int one_plus, float eps);
int xalm_cuda_dual_norm_hyper(float* xs, const float* a, const float* b, const float* wa, const float* wb, float eps, int S, int T, int W,
                              const float* mix, const float* out_coef, const float* scale);
int xalm_cuda_glu_rows(float* out, const float* x, const float* w_gate, const float* w_up, int T, int ff, int K, float limit, float alpha, int w_bf16);
/* swa_attention_kept: the same window, but every position j < keep_first stays visible to all later queries (at its true position); the
 *   cache holds those in slots of their own and the rest in a ring of `ring` slots.  No soft cap, bias, mixing or gate.
 * group_norm_residual: x_out = x_in + gnorm(sum_k part_w[t, k] y[t * parts + k]) * w, gnorm = RMS norm over each of `groups` equal parts of
 *   the row (x_in NULL: no residual; part_w NULL: parts == 1).  With dwa (n_hist + 1 coefficients) and hist (n_hist, T, W):
 *   avg_out = sum_j dwa[j] hist[j] + dwa[n_hist] x_out.
 * qkv_post: rows of [q (H d) | k (G d) | v (G dv)] for positions pos0..: bias, rotation of the first 2 rot_half dimensions of every q / k head
 *   (dimension i with i + rot_half, angle = position * freq[i]), then weightless RMS norms of q, k heads (norm_qk) and v heads (norm_v).
 *   q_out (T, H d); k_out / v_out: the whole cache (keep_first + ring slots), position p in slot p (p < keep_first) or
 *   keep_first + (p - keep_first) % ring.
 * delta_rule: T tokens of the gated delta rule.  q, k (T, G d) and v (T, H dv) are the projections BEFORE the causal convolutions
 *   (weights (channels, taps), last column = the current token) and silu; q and k heads are then scaled to unit length
 *   (x / sqrt(sum x^2 + unit_eps); q times q_scale); beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias)); per head
 *   S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q; out = o / rms(o) * norm_w * silu(gate).  state (H, d, dv) and conv_state
 *   (taps - 1, 2 G d + H dv: the last inputs of the q | k | v channels, oldest first) are read and written.
 * moe_ffn: router scores s = sigmoid(h W_router^T); with n_groups > 1 the experts form equal groups of neighbours, a group scores the sum of its
 *   two largest s and only the keep_groups best groups can be chosen from; idx / wgt (T, top) = the chosen experts and their scores;
 *   out_pairs (T * top, K) = W_down[e] (act(W_gate[e] h) * (W_up[e] h)) for every chosen (token, expert); act: 1 silu, 2 tanh-gelu. */
int xalm_cuda_swa_attention_kept(float* out, const float* q, const float* k, const float* v, int T, int pos0, int H, int G, int d, int dv, int window,
                                 int keep_first, float scale, int ring, int n_splits, int cache_bf16);
int xalm_cuda_group_norm_residual(float* x_out, float* avg_out, const float* y, int parts, const float* part_w, const float* w, int groups, float eps,
                                  const float* x_in, const float* hist, int n_hist, const float* dwa, int T, int W);
int xalm_cuda_qkv_post(float* q_out, float* k_out, float* v_out, const float* proj, int T, int pos0, int H, int G, int d, int dv, const float* bq,
                       const float* bk, const float* bv, const float* freq, int rot_half, int norm_qk, int norm_v, float eps, int keep_first, int ring);
int xalm_cuda_delta_rule(float* out, float* state, float* conv_state, const float* q, const float* k, const float* v, const float* gate, const float* b,
                         const float* a_in, int T, int H, int G, int d, int dv, int taps, const float* wq, const float* wk, const float* wv,
                         const float* A_log, const float* dt_bias, const float* norm_w, float eps, float unit_eps, float q_scale);
int xalm_cuda_moe_ffn(float* out_pairs, int* idx, float* wgt, const float* h, const float* w_router, const float* w_gate, const float* w_up,
                      const float* w_down, int T, int K, int E, int top, int ff, int n_groups, int keep_groups, int act, int w_bf16);

/* Mechanisms of the latent-attention / retention designs, as ops (host arrays in and out, the same kernels the families run):
 * moe_ffn_routed: moe_ffn with the router's variants.  score_kind 0: sigmoid, 1: softmax over all experts; group_kind 0: a group scores the
 *   sum of its two largest s, 1: its largest; renormalise 1: the chosen scores over (their sum + 1e-20); act 0: the clamped gate
 *   min(g, limit) sigmoid(1.702 .) (clamp(u, +-limit) + 1), 1 silu, 2 tanh-gelu; x_io (T, K) or NULL: x_io += sum over a token's slots of
 *   wgt * out_pairs.
 * retention: per head S <- decay[h] S + (k_scale k_t) v_t^T, o_t = S^T q_t for T tokens from position pos0; q and k (T, H d) are turned first
 *   (the first 2 rot_half entries of a head, entry i with i + rot_half, angle = position * freq[i]); o over its root mean square (eps, no
 *   weight), times silu(gate) when gate (T, H dv) is given.  state (H, d, dv) is read and written.
 * latent_post: proj (T, q_rank + kv_rank + rot) -> cq_out (T, q_rank) = rmsnorm(proj[:, :q_rank]) q_norm; cache row of position p (slot
 *   p % ring of cache_out (ring, kv_rank + rot)) = [rmsnorm(kv latent) kv_norm | the rot shared key entries turned by p].
 * latent_attend: causal softmax attention of H heads over cache rows (pos0 + T, ld) whose first R entries are the latent c and next r the
 *   turned shared key: score = scale (q_h[:d] . (uk_h c) + turn(q_h[d:]) . k_rot), out_h = uv_h (sum_j p_j c_j), times sigmoid(gate) when
 *   given.  q (T, H (d + r)) un-turned, uk (H d, R), uv (H dv, R).  n_splits 0: the launcher chooses.
 * rows_act: out = act(x W^T) (act 1 relu squared, 2 sigmoid, 3 silu) or, with act 0, cap * tanh(x W^T / cap) (cap > 0) times mul_act(mul). */
int xalm_cuda_moe_ffn_routed(float* out_pairs, int* idx, float* wgt, float* x_io, const float* h, const float* w_router, const float* w_gate,
                             const float* w_up, const float* w_down, int T, int K, int E, int top, int ff, int n_groups, int keep_groups, int act,
                             int w_bf16, int score_kind, int group_kind, int renormalise, float limit);
int xalm_cuda_retention(float* out, float* state, const float* q, const float* k, const float* v, const float* gate, int T, int pos0, int H, int d, int dv,
                        const float* decay, const float* freq, int rot_half, float k_scale, float eps);
int xalm_cuda_latent_post(float* cq_out, float* cache_out, const float* proj, int T, int pos0, int q_rank, int kv_rank, int rot, const float* q_norm,
                          const float* kv_norm, const float* freq, float eps, int ring, int cache_bf16);
int xalm_cuda_latent_attend(float* out, const float* q, const float* cache, const float* gate, int T, int pos0, int H, int d, int r, int dv, int R, int ld,
                            const float* uk, const float* uv, const float* freq, float scale, int n_splits, int cache_bf16, int w_bf16);
int xalm_cuda_rows_act(float* out, const float* x, const float* w, int T, int N, int K, int act, float cap, const float* mul, int mul_act, int w_bf16);

/* Mechanisms of designs with convolved readers, keyed recurrences and sink attention, as ops (host arrays in and out, the same kernels):
 * norm_conv: for each of `readers` (1 or 2) readers r of the same rows x (T, W): h = grouped RMS norm of x (groups equal parts, each over
 *   its own sqrt(mean + eps)) times w[r], out[r] = h + causal depthwise convolution of h over time with cw[r] (W, taps), last column = the
 *   current row.  hist (readers, taps - 1, W): the normed rows before x[0], oldest first; rewritten with the last taps - 1 normed rows.
 * short_conv: out[t, c] = act(bias[c] + sum_j w[c, j] x[t - taps + 1 + j, c]) (act 0 none, 3 silu), hist (taps - 1, C) raw inputs as above.
 * embed_pair: out[t] = grouped norm(table[token_t] * scale + pair[(token_{t-1} * mul_prev + token_t * mul_cur) mod buckets]) * w, the row
 *   `buckets` of pair where there is no previous token (prev < 0 for t = 0); pair NULL: no pair rows; w NULL: no norm.
 * keyed_recurrence: per head S_t = diag(f_t) S_{t-1} + (s_t k_t) v_t^T, o_t = S_t^T (q_scale q_t) + skip[h] v_t; q, k (T, H / rep * d) shared by
 *   `rep` neighbouring heads.  mode 1: f (T, H d) decays as they are, s = 1.  mode 2: f (T, H) raw step sizes, dt = softplus(f + dt_bias[h]),
 *   decay exp(-exp(A_log[h]) dt) on every channel, s = dt.  Then, when given: o over its root mean square times norm_w (dv), times silu(gate).
 * sink_attention: causal softmax attention of H heads over G key heads whose denominator also holds exp(sink[h]); result times out_scale
 *   (0: 1).  k (pos0 + T, G d), v (pos0 + T, G dv).
 * qk_post: proj (T, (H + G) d) = [q | k]; q_out = turned q; k_out (ring, G d) the turned keys and v_out (ring, G d) the keys as they came, row
 *   p % ring for position p.  Turn: the first 2 rot_half entries of a head, entry i with i + rot_half, by p * freq[i], cos and sin times rot_mag.
 * rows_act_bias: out = act(x W^T + bias); act as rows_act, 4 tanh-gelu, 5 sigmoid(.)^act_pow.
 * gated_group_norm: out[:, :W] of rows ld_out wide = grouped RMS norm of y * silu(gate) (gate NULL: of y), times w, times out_scale (0: 1). */
int xalm_cuda_norm_conv(float* out, float* hist, const float* x, int T, int W, int groups, int taps, int readers, const float* w, const float* cw, float eps);
int xalm_cuda_short_conv(float* out, float* hist, const float* x, int T, int C, int taps, const float* w, const float* bias, int act);
int xalm_cuda_embed_pair(float* out, const int* tokens, int T, int prev, const float* table, int vocab, const float* pair, int buckets, int mul_prev,
                         int mul_cur, float scale, const float* w, int groups, int W, float eps);
int xalm_cuda_keyed_recurrence(float* out, float* state, const float* q, const float* k, const float* v, const float* f, int T, int H, int rep, int d, int dv,
                               int mode, float q_scale, const float* dt_bias, const float* A_log, const float* skip, const float* norm_w, const float* gate,
                               float eps);
int xalm_cuda_sink_attention(float* out, const float* q, const float* k, const float* v, int T, int pos0, int H, int G, int d, int dv, float scale,
                             const float* sink, float out_scale, int n_splits, int cache_bf16);
int xalm_cuda_qk_post(float* q_out, float* k_out, float* v_out, const float* proj, int T, int pos0, int H, int G, int d, const float* freq, int rot_half,
                      float rot_mag, int ring);
int xalm_cuda_rows_act_bias(float* out, const float* x, const float* w, int T, int N, int K, int act, const float* bias, float act_pow, int w_bf16);
int xalm_cuda_gated_group_norm(float* out, const float* y, const float* gate, const float* w, int T, int W, int groups, float eps, float out_scale, int ld_out);

/* Tensor parallel plumbing (no reference analogue; north star).  Rank 0 makes an id, the host side ships it to
 * the other ranks (torch.distributed / MPI / a file), every rank calls comm_init before finalize. */
#define XALM_COMM_ID_BYTES 128
int xalm_cuda_comm_unique_id(void* id128);
int xalm_cuda_comm_init(xalm_cuda_model* m, const void* id128);

/* Optional: one-shot allreduce over NVLink peer memory instead of NCCL for the two per-layer exchanges.  Every rank exports
 * a CUDA IPC handle of its exchange buffer, the host gathers all of them (rank order) and hands the table to every rank.
 * Call after create and before finalize; without it the backend uses ncclAllReduce. */
#define XALM_IPC_HANDLE_BYTES 64
int xalm_cuda_ipc_export(xalm_cuda_model* m, void* handle64);
int xalm_cuda_ipc_import(xalm_cuda_model* m, const void* handles /* tp_size x 64 bytes */);

/* Run on a caller-provided cudaStream_t (e.g. the framework's current stream) instead of the model's own. */
int xalm_cuda_set_stream(xalm_cuda_model* m, void* cuda_stream);

/* ---- forward: Model::forward(state, token, pos, mode)  (model.h:272, infer.cpp:604-638) ---------------- */
/* Synchronous: on return with mode == XALM_OUTPUT_LOGITS, `logits_host` (vocab_size floats, caller-owned,
 * may be pageable) holds what InferenceState::logits() would.  logits_host may be NULL (leave them on device). */
int xalm_cuda_forward(xalm_cuda_model* m, int token, int pos, int mode, float* logits_host);
/* forward(OUTPUT_LOGITS) followed by Sampler::sample_argmax (sampler.cpp:3-16, FLT_MIN-seeded running maximum, first
 * maximum wins) on the device: only the 4-byte token id crosses PCIe.  Leaves the host logits buffer untouched. */
int xalm_cuda_forward_argmax(xalm_cuda_model* m, int token, int pos, int* next_token);
/* Enqueue only (no host sync, logits stay on the device): the device-timed leg of bench.py. */
int xalm_cuda_forward_async(xalm_cuda_model* m, int token, int pos, int mode);
int xalm_cuda_sync(xalm_cuda_model* m);
/* ---- batched prefill: the loops of main.cpp:94-100 (prompt hydrate) and :244-254 (perplexity), which call
 *      Model::forward once per position, as ONE pass over the weights on the tcgen05 tensor-core path ---------- */
/* Positions pos0 .. pos0+n-1 (pos0 + n <= max_seq_len: no ring wrap; past that use xalm_cuda_forward).  Fills the KV
 * cache exactly as n forward calls would (fp16-operand rounding aside).  want_logits: 0 = none (HYDRATE_KV_CACHE for
 * every position), 1 = logits of the last position -> logits_host[vocab], 2 = every position -> logits_host[n*vocab].
 * targets/probs_host (n entries each, or NULL; needs want_logits 2): probs_host[i] = Sampler::sample_prob(targets[i])
 * on the logits of position pos0+i (sampler.cpp:18-33) — what perplexity mode takes the log of (main.cpp:251).
 * logits_host may be NULL.  Synchronous.  Tensor-core operands are fp16 with fp32 accumulation; the "prefill_split"
 * knob (xalm_cuda_tune) picks how fp32 values enter them: 3 (default) = hi+lo fp16 pairs for activations, weights and the
 * attention operands (3 MMAs per product; 32-layer 4k-token logits within ~1e-3 of the token-at-a-time path), 2 = pairs
 * for activations only, 1 = plain fp16 (fastest; ~4e-2 at that depth).  North star tolerance: 1e-2. */
int xalm_cuda_prefill(xalm_cuda_model* m, const int* tokens, int n, int pos0, int want_logits, float* logits_host,
                      const int* targets, float* probs_host);
/* Enqueue only (no read-back, no host sync) — bench.py's device-timed leg. */
int xalm_cuda_prefill_async(xalm_cuda_model* m, const int* tokens, int n, int pos0, int want_logits);
/* Pinned host buffer the logits are copied into by xalm_cuda_forward (alias it as InferenceState::_logits). */
float* xalm_cuda_logits_host(xalm_cuda_model* m);
/* Model::active_bytes(pos) (model.cpp:12-35), 64-bit, per-format bytes; this rank's shard only. */
int xalm_cuda_active_bytes(xalm_cuda_model* m, long long pos, long long* bytes);
/* Kernels launched by the last forward (bench.py's gpu_launches). */
int xalm_cuda_last_launch_count(xalm_cuda_model* m, int* n);

/* ---- state read-back for parity tests (InferenceState accessors model.h:124-139, Block KV model.h:222-223) -- */
enum xalm_state_buf { XALM_S_X = 0, XALM_S_XB = 1, XALM_S_XB2 = 2, XALM_S_HB = 3, XALM_S_Q = 5, XALM_S_LOGITS = 9 };
int xalm_cuda_read_state(xalm_cuda_model* m, int which, float* dst, size_t n);
/* which: 0 = key_cache, 1 = value_cache; fp16 bits, (max_seq_len, local kv_dim) */
int xalm_cuda_read_kv(xalm_cuda_model* m, int layer, int which, uint16_t* dst, size_t n_elems);

/* ---- op-level entry points: the functions model.h:286-316 exposes "for tests", host pointers in and out ---- */
/* Type::get_float over a buffer (types.h:406-427) / quants.py dequantize: n_elems elements -> fp32. */
int xalm_cuda_dequant(int type_id, const void* src, size_t n_elems, float* dst);
/* matmul(xout, x, w, n, d) (model.h:315, infer.cpp:185-216): W(d,n) row-major in on-disk bytes of `type_id`. */
int xalm_cuda_matmul(float* xout, const float* x, const void* w, int type_id, int n, int d);
/* mha_cuda — the prototype the reference declares and never defines (model.h:308-313). att may be NULL. */
int xalm_cuda_mha(float* xout, float* att, const uint16_t* kb, const uint16_t* vb, const float* q, int head_dim,
                  int kv_len, int max_seq_len, int n_heads, int n_kv_heads);
/* The batched form of matmul: out(T,N) = a(T,K) . W(N,K)^T on the tcgen05 path (dequantise to fp16 tiles, UMMA, fp32
 * accumulate).  split: 1 = fp16 activations, 2 = hi+lo fp16 pair. */
int xalm_cuda_gemm(float* out, const float* a, const void* w, int type_id, int T, int K, int N, int split);
/* rmsnorm(o, x, weight, size, eps) (infer.cpp:224-251); weight F32 or BF16 only. */
int xalm_cuda_rmsnorm(float* o, const float* x, const void* weight, int weight_type, int size, float eps);
/* rope(vec, d, head_dim, pos, theta, rotary_dim) (infer.cpp:305-322), in place. */
int xalm_cuda_rope(float* vec, int d, int head_dim, int pos, float theta, int rotary_dim);
/* ffn: hb = act(W1 x) * (W3 x); xout = W2 hb   (ffn_cpu, infer.cpp:519-551) with weights of `type_id`. */
int xalm_cuda_ffn(float* xout, const float* x, const void* w1, const void* w2, const void* w3, int type_id,
                  int hidden_dim, int dim, int act);

/* Integer tuning knobs by name ("pdl", "graph", "attn_splits", "attn_min_split", "mv_cfg_rows", "prefill_split", "idp", "mma", "mega",
 * "tail_prefetch_mb", ...); an XALM_<KEY> environment variable overrides the stored value.  Takes effect for graphs captured
 * afterwards; "mma" (which matvec kernel and device layout the integer formats take: 0 = dp4a + unit layout, 1 = tensor-core mma +
 * fragment tiles, 2 = default: mma for the 4/5-bit formats and, under tensor parallelism, the 8-bit ones) and "mega" are read when a
 * matrix is uploaded. */
int xalm_cuda_tune(const char* key, int value);

/* In-kernel timeline (there is no nsys here): with out == NULL start recording up to n_records kernels; with out != NULL
 * stop and fetch the records — 4 x u64 each: kernel id (100+epi = TMA matvec, 200+epi = LDG matvec, 300 = attention),
 * %globaltimer (ns) of block 0 at entry, after the dependency wait, at exit. */
int xalm_cuda_timeline(int n_records, unsigned long long* out, int* n_out);
/* Same idea for the one-kernel-per-token decode path (decode_mega.cu; tune "mega_timeline" = 1 before the first forward):
 * out receives n_phases x 8 u64 of CTA 0 (phase entry, hand-off done, activations staged, phase done, four finer marks) followed by
 * n_phases x grid arrival stamps of every CTA.  With out == NULL only n_phases / grid are returned (0 = token kernel not in use). */
int xalm_cuda_mega_timeline(xalm_cuda_model* m, unsigned long long* out, size_t cap_words, int* n_phases, int* grid);

/* ---- kernel micro-benchmark hook (bench.py roofline leg; README.md:62-84 `-k matmul`) ------------------- */
/* Times `iters` back-to-back launches of the matvec kernel on resident weights of `type_id` (random bytes), rotating
 * over `n_buffers` distinct copies so the working set exceeds L2.  epi: 0 = plain store of d outputs from a (d,n) matrix,
 * 2 = the fused gate|up kernel (2d rows -> d outputs through act*gate); with_norm: fuse the rmsnorm prologue.  Returns
 * mean milliseconds per launch (CUDA events on the launch stream). */
int xalm_cuda_bench_matvec(int type_id, int n, int d, int epi, int with_norm, int n_buffers, int iters, float* ms_per_launch);

/* Times `iters` launches of the tcgen05 GEMM kernel alone on resident fp16 tiles (T x K activations, N x K weights);
 * mean milliseconds per launch.  2*T*N*K flops per launch. */
int xalm_cuda_bench_gemm(int T, int N, int K, int split, int iters, float* ms_per_launch);

#ifdef __cplusplus
}
#endif
#endif /* XALM_CUDA_H */
