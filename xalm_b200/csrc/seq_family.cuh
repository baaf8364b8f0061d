// seq_family.cuh — the sequence engine shared by the model families that a config.json describes (Nabalix, Bolovik, Duletar, Kubolorn): what a
// family does NOT write itself.
//
//   * tensors by name: the family lists what it reads (expect), the loader uploads them (any order, fp32 / fp16 / bf16), finalize
//     turns them into device layouts (upload_rows: several matrices stacked or interleaved into one; upload_vec);
//   * the step function (seq_step): n tokens of the running sequence from the position the sequence stands at, cut into passes of at
//     most "seq_chunk" positions; one-token steps replay a captured CUDA graph whose position and token live in device memory;
//   * row products (rows_product): the fp32 FMA kernels of mix_ops.cuh with a fused epilogue, or, for passes of many tokens in the
//     16-bit mode, the tcgen05 GEMM of prefill.cu on the weight's resident fp16 tiles followed by the same epilogue;
//   * release (the sequence is over: the family zeroes its state, the position returns to 0), logits read-back, target
//     probabilities, launch counts, the table of C entry points (seq_family_table).
//
// A family derives its model struct from SeqModel and fills a SeqHooks: parse_config (sizes and expected tensors), finalize (its
// device layouts, caches and state), enqueue_pass (the kernels of one pass), release, active_bytes, state_buffer, destroy.
// Everything here has internal linkage: each family's translation unit gets its own copy.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <string>
#include <vector>

#ifndef XALM_SECONDARY_TU
#define XALM_SECONDARY_TU // the Llama family's translation unit owns the shared non-inline definitions
#endif
#include "common.cuh"
#include "family.h"
#include "formats.cuh"
#include "host/json.h"
#include "mix_ops.cuh"
#include "prefill.h"

namespace xalm {
namespace seq {

using namespace mix;

// a tensor as uploaded: fp32 on the host until finalize builds the device layouts
struct HostTensor {
	std::vector<int> shape;
	bool required = true;
	bool matrix = false;
	bool got = false;
	int type = 0;
	std::vector<float> v;
};

struct SeqModel;
struct SeqHooks {
	int (*parse_config)(SeqModel*, const char* json);        // sizes, constants, expected tensors; touches no device
	int (*finalize)(SeqModel*);                              // the family's device layouts, cache, state and pass buffers
	int (*enqueue_pass)(SeqModel*, int n, int want, int* nl); // kernels of one pass of n <= chunk tokens (ids in d_tokens, position in d_step);
	                                                         // want: 0 no logits, 1 the last row's, 2 every row's -> m->logits
	int (*release)(SeqModel*);                               // enqueue on m->stream whatever gives the sequence's state back
	long long (*active_bytes)(SeqModel*, long long pos);     // bytes a one-token step at `pos` reads beyond weight_bytes' matrices
	bool (*state_buffer)(SeqModel*, int layer, const float** src, size_t* count); // recurrent state of a layer, for read_state(1000 + layer)
	void (*destroy)(SeqModel*);                              // frees what finalize made outside m->allocs, then deletes the model
};

struct SeqModel { // what a handle of these families points to (ModelHead first)
	ModelHead head = {nullptr};
	const SeqHooks* hooks = nullptr;
	int device = 0, precision = XALM_PRECISION_BF16, max_tokens = 0;
	int vocab = 0, width = 0, n_layers = 0;
	float eps = 1e-5f;
	std::map<std::string, HostTensor> tensors;
	std::vector<std::string> order; // expected tensors in file order
	bool w_bf16 = true;             // matrices live on the device as bf16 (else fp32)
	bool finalized = false;
	std::vector<void*> allocs;
	void *embed = nullptr, *w_head = nullptr;
	WMat m_head;
	TcWeight t_head;
	uint8_t *a_hi = nullptr, *a_lo = nullptr; // activation operand planes of the tensor-core path
	float* tc_out = nullptr;                  // its plain fp32 product, when an epilogue follows
	size_t tc_a_bytes = 0, tc_cols = 4;       // what the registered weights need of them
	int tc_min_rows = 32;
	float* final_norm = nullptr;
	int chunk = 256;                          // most positions of one pass
	float *logits = nullptr, *layer_sums = nullptr;
	int keep_layers = 0;                      // keep the residual stream after every layer of the last pass (read_state(100 + layer))
	int graph_launches[2] = {0, 0};           // kernels in the captured one-token step (without / with logits)
	int* d_tokens = nullptr;
	SeqStep* d_step = nullptr;
	float* h_logits = nullptr; // pinned, chunk x vocab
	cudaStream_t stream = nullptr, own_stream = nullptr;
	cudaStream_t side = nullptr; // for mixers of a layer that do not depend on one another
	cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
	cudaGraphExec_t graph[2] = {nullptr, nullptr};
	int pos = 0; // tokens the running sequence holds
	int prev_token = -1; // the last of them (-1: none yet), handed to the kernels as SeqStep.prev
	int last_launches = 0;
	bool use_tc = false;
	long long weight_bytes = 0, weight_bytes_tc = 0;
};

namespace {

// ---- config.json helpers --------------------------------------------------------------------------------------------------------
int geti(const xjson::Value& o, const char* k) {
	const xjson::Value& v = o.at(k);
	if (v.kind != xjson::Value::Number) throw std::invalid_argument(std::string("config: '") + k + "' is not a number");
	return (int) v.num;
}
double getf(const xjson::Value& o, const char* k) {
	const xjson::Value& v = o.at(k);
	if (v.kind != xjson::Value::Number) throw std::invalid_argument(std::string("config: '") + k + "' is not a number");
	return v.num;
}
void expect(SeqModel* m, const std::string& name, std::vector<int> shape, bool matrix, bool required = true) {
	HostTensor t;
	t.shape = std::move(shape);
	t.matrix = matrix;
	t.required = required;
	m->tensors.emplace(name, std::move(t));
	m->order.push_back(name);
}
const HostTensor* tensor_or_null(SeqModel* m, const std::string& n) {
	const HostTensor& t = m->tensors.at(n);
	return t.got ? &t : nullptr;
}

// ---- device memory --------------------------------------------------------------------------------------------------------------
template <typename T>
int dev_alloc(SeqModel* m, T** p, size_t count, bool zero = false) {
	void* q = nullptr;
	const size_t bytes = std::max<size_t>(count * sizeof(T), 16);
	cudaError_t e = cudaMalloc(&q, bytes);
	if (e != cudaSuccess) return set_error(XALM_ERR_CUDA, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
	m->allocs.push_back(q);
	if (zero) XALM_CUDA_CHECK(cudaMemset(q, 0, bytes));
	*p = reinterpret_cast<T*>(q);
	return XALM_OK;
}

int upload_floats(SeqModel* m, const float* src, size_t n, float** dst) {
	XALM_TRY(dev_alloc(m, dst, n));
	XALM_CUDA_CHECK(cudaMemcpy(*dst, src, n * 4, cudaMemcpyHostToDevice));
	m->weight_bytes += (long long) n * 4;
	return XALM_OK;
}

int upload_vec(SeqModel* m, const std::string& name, float** dst) { // absent optional tensors leave NULL
	*dst = nullptr;
	const HostTensor& t = m->tensors.at(name);
	if (!t.got) return XALM_OK;
	return upload_floats(m, t.v.data(), t.v.size(), dst);
}

uint16_t f32_to_bf16_bits(float f) {
	uint32_t u;
	memcpy(&u, &f, 4);
	if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t) ((u >> 16) | 0x40);
	u += 0x7fffu + ((u >> 16) & 1u);
	return (uint16_t) (u >> 16);
}

// rows of several host matrices, one after the other, as one device matrix (bf16 or fp32, as the model keeps its matrices).
// interleave: the parts are taken in consecutive pairs whose rows alternate (gate / up of a gated feed-forward, one pair per expert).
// NULL parts are skipped.
int upload_rows(SeqModel* m, const std::vector<const HostTensor*>& parts, int K, bool interleave, void** dst, WMat* wm) {
	size_t rows = 0;
	for (const HostTensor* t : parts) rows += t ? (size_t) t->shape[0] : 0;
	const size_t esz = m->w_bf16 ? 2 : 4;
	std::vector<uint8_t> buf(rows * (size_t) K * esz);
	size_t r = 0;
	auto put_row = [&](const float* src) {
		if (m->w_bf16) {
			uint16_t* o = reinterpret_cast<uint16_t*>(buf.data()) + r * (size_t) K;
			for (int k = 0; k < K; k++) o[k] = f32_to_bf16_bits(src[k]);
		} else memcpy(buf.data() + r * (size_t) K * 4, src, (size_t) K * 4);
		r++;
	};
	if (interleave) {
		for (size_t p = 0; p + 1 < parts.size(); p += 2)
			for (int i = 0; i < parts[p]->shape[0]; i++) {
				put_row(parts[p]->v.data() + (size_t) i * K);
				put_row(parts[p + 1]->v.data() + (size_t) i * K);
			}
	} else {
		for (const HostTensor* t : parts)
			if (t)
				for (int i = 0; i < t->shape[0]; i++) put_row(t->v.data() + (size_t) i * K);
	}
	uint8_t* d = nullptr;
	XALM_TRY(dev_alloc(m, &d, buf.size() + 64));
	XALM_CUDA_CHECK(cudaMemcpy(d, buf.data(), buf.size(), cudaMemcpyHostToDevice));
	*dst = d;
	m->weight_bytes += (long long) buf.size();
	if (wm) {
		*wm = WMat();
		wm->type = m->w_bf16 ? XALM_BF16 : XALM_F32;
		wm->rows = (int) rows;
		wm->n = K;
		wm->p0 = d;
		wm->s0 = (size_t) K * esz;
	}
	return XALM_OK;
}

// tensor-core operands: a matrix whose shape the GEMM takes keeps its fp16 tiles beside the rows the one-token steps stream
int tc_register(SeqModel* m, const WMat& wm, TcWeight* t) {
	if (!m->use_tc || !tc_shape_ok(wm.rows, wm.n, wm.rows)) return XALM_OK; // this one stays on the fp32 kernels
	XALM_TRY(tc_weight_build(wm, 1, t, m->stream));
	m->tc_a_bytes = std::max(m->tc_a_bytes, tc_a_plane_bytes(m->chunk, wm.n));
	m->tc_cols = std::max(m->tc_cols, (size_t) wm.rows);
	m->weight_bytes_tc += (long long) t->NT * t->KT * 256 * 64 * 2;
	return XALM_OK;
}

// ---- row products ---------------------------------------------------------------------------------------------------------------
// Passes of few tokens and the fp32 mode: the fp32 FMA kernels of mix_ops.cuh with the epilogue fused.  Passes of tc_min_rows tokens
// or more in the 16-bit mode: the tcgen05 GEMM of prefill.cu on the weight's resident fp16 tiles (activations packed to fp16, one
// plane, or hi + lo with "seq_tc" = 2), fp32 accumulation, then the same epilogue as an elementwise kernel.
int rows_product(SeqModel* m, const float* A, int lda, const void* W, const TcWeight* tw, int T, int N, int K, const RowsEpi& e, int* nl) {
	if (m->use_tc && tw && tw->hi && T >= m->tc_min_rows && lda == K) {
		if (e.kind == EPI_STORE && e.ldo % 4 == 0 && e.cap == 0.f && !e.mul) { // nothing to do to the product: the GEMM stores it itself
			*nl += 2;
			return tc_gemm(*tw, A, T, e.out, e.ldo, m->a_hi, m->a_lo, m->stream);
		}
		*nl += 3;
		XALM_TRY(tc_gemm(*tw, A, T, m->tc_out, N, m->a_hi, m->a_lo, m->stream));
		return launch_rows_epilogue(m->tc_out, N, T, N, e, m->stream);
	}
	(*nl)++;
	return launch_rows(A, lda, W, m->w_bf16, T, N, K, e, m->stream);
}

#define XALM_SEQ_LAUNCH_CHECK(what)                                                                                  \
	do {                                                                                                            \
		(*nl)++;                                                                                                    \
		cudaError_t e_ = cudaGetLastError();                                                                        \
		if (e_ != cudaSuccess) return set_error(XALM_ERR_CUDA, what " launch failed: %s", cudaGetErrorString(e_));   \
	} while (0)

// ---- the step function ----------------------------------------------------------------------------------------------------------
int check_ready(SeqModel* m) {
	if (!m) return set_error(XALM_ERR_INVALID, "model is NULL");
	if (!m->finalized) return set_error(XALM_ERR_STATE, "the model is not finalized");
	XALM_CUDA_CHECK(cudaSetDevice(m->device));
	return XALM_OK;
}

int ensure_graph(SeqModel* m, int mode) {
	if (m->graph[mode]) return XALM_OK;
	cudaGraph_t g = nullptr;
	XALM_CUDA_CHECK(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
	int nl = 0;
	const int rc = m->hooks->enqueue_pass(m, 1, mode ? 1 : 0, &nl);
	cudaError_t e = cudaStreamEndCapture(m->stream, &g);
	if (rc != XALM_OK) {
		if (g) cudaGraphDestroy(g);
		return rc;
	}
	if (e != cudaSuccess) return set_error(XALM_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
	m->graph_launches[mode] = nl;
	e = cudaGraphInstantiate(&m->graph[mode], g, 0);
	cudaGraphDestroy(g);
	if (e != cudaSuccess) return set_error(XALM_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
	return XALM_OK;
}

// one pass of n <= chunk tokens at the sequence's position; the logits (want) stay on the device
int run_pass(SeqModel* m, const int* tokens, int n, int want) {
	for (int i = 0; i < n; i++)
		if (tokens[i] < 0 || tokens[i] >= m->vocab) return set_error(XALM_ERR_INVALID, "token %d out of range", tokens[i]);
	const SeqStep st = {m->pos, n, m->prev_token};
	XALM_CUDA_CHECK(cudaMemcpyAsync(m->d_tokens, tokens, (size_t) n * 4, cudaMemcpyHostToDevice, m->stream));
	XALM_CUDA_CHECK(cudaMemcpyAsync(m->d_step, &st, sizeof st, cudaMemcpyHostToDevice, m->stream));
	int nl = 0;
	if (n == 1 && tune("seq_graph")) {
		const int mode = want ? 1 : 0;
		XALM_TRY(ensure_graph(m, mode));
		XALM_CUDA_CHECK(cudaGraphLaunch(m->graph[mode], m->stream));
		nl = m->graph_launches[mode]; // as counted at capture
	} else {
		XALM_TRY(m->hooks->enqueue_pass(m, n, want, &nl));
	}
	m->last_launches = nl;
	m->pos += n;
	m->prev_token = tokens[n - 1];
	return XALM_OK;
}

// n tokens of the running sequence from position pos0 (= what the sequence holds)
int seq_step(SeqModel* m, const int* tokens, int n, int pos0, int want, float* logits_host, const int* targets, float* probs_host) {
	XALM_TRY(check_ready(m));
	if (!tokens || n <= 0) return set_error(XALM_ERR_INVALID, "step: no tokens");
	if (want < 0 || want > 2) return set_error(XALM_ERR_INVALID, "step: want_logits = %d", want);
	if (targets && want != 2) return set_error(XALM_ERR_INVALID, "step: target probabilities need the logits of every position");
	if (pos0 != m->pos)
		return set_error(XALM_ERR_STATE, "step: position %d, but the sequence holds %d tokens (release it to start another)", pos0, m->pos);
	if ((long long) pos0 + n > m->max_tokens) return set_error(XALM_ERR_INVALID, "step: positions [%d, %d) exceed max_tokens %d", pos0, pos0 + n, m->max_tokens);
	const int V = m->vocab;
	for (int at = 0; at < n; at += m->chunk) {
		const int nc = std::min(m->chunk, n - at);
		const bool last = at + nc == n;
		const int w = want == 2 ? 2 : (want == 1 && last ? 1 : 0);
		XALM_TRY(run_pass(m, tokens + at, nc, w));
		if (w) {
			const int rows = w == 2 ? nc : 1;
			XALM_CUDA_CHECK(cudaMemcpyAsync(m->h_logits, m->logits, (size_t) rows * V * 4, cudaMemcpyDeviceToHost, m->stream));
			XALM_CUDA_CHECK(cudaStreamSynchronize(m->stream));
			if (logits_host) memcpy(logits_host + (w == 2 ? (size_t) at * V : 0), m->h_logits, (size_t) rows * V * 4);
			if (targets && probs_host)
				for (int i = 0; i < rows; i++) { // Sampler::sample_prob (sampler.cpp:18-33)
					const float* lg = m->h_logits + (size_t) i * V;
					if (targets[at + i] < 0 || targets[at + i] >= V) return set_error(XALM_ERR_INVALID, "step: target %d out of range", targets[at + i]);
					float top = lg[0];
					for (int k = 1; k < V; k++) top = std::max(top, lg[k]);
					float den = 0.f;
					for (int k = 0; k < V; k++) den += expf(lg[k] - top);
					probs_host[at + i] = expf(lg[targets[at + i]] - top) / den;
				}
		}
	}
	XALM_CUDA_CHECK(cudaStreamSynchronize(m->stream));
	return XALM_OK;
}

// ---- entry points of the family table ---------------------------------------------------------------------------------------------
void seq_destroy(SeqModel* m) {
	if (!m) return;
	cudaSetDevice(m->device);
	if (m->stream) cudaStreamSynchronize(m->stream);
	for (int i = 0; i < 2; i++)
		if (m->graph[i]) cudaGraphExecDestroy(m->graph[i]);
	for (void* p : m->allocs) cudaFree(p);
	tc_weight_free(&m->t_head);
	if (m->h_logits) cudaFreeHost(m->h_logits);
	if (m->own_stream) cudaStreamDestroy(m->own_stream);
	if (m->side) cudaStreamDestroy(m->side);
	if (m->ev_fork) cudaEventDestroy(m->ev_fork);
	if (m->ev_join) cudaEventDestroy(m->ev_join);
	m->hooks->destroy(m);
}

// M: the family's model struct (derived from SeqModel)
template <typename M>
int seq_create(const ModelFamily* family, const SeqHooks* hooks, const char* json, int device, int max_tokens, int precision, xalm_cuda_model** out) {
	if (max_tokens <= 0) return set_error(XALM_ERR_INVALID, "max_tokens must be positive");
	M* mm = new M();
	SeqModel* m = mm;
	m->head.family = family;
	m->hooks = hooks;
	m->device = device;
	m->precision = precision;
	m->max_tokens = max_tokens;
	const int rc = hooks->parse_config(m, json); // before the device is touched: a bad config is reported as such on any machine
	if (rc != XALM_OK) { delete mm; return rc; }
	int ndev = 0;
	cudaError_t e = cudaGetDeviceCount(&ndev);
	if (e != cudaSuccess) { delete mm; return set_error(XALM_ERR_CUDA, "cudaGetDeviceCount failed: %s", cudaGetErrorString(e)); }
	if (device < 0 || device >= ndev) { delete mm; return set_error(XALM_ERR_CUDA, "device %d not available (%d devices)", device, ndev); }
	e = cudaSetDevice(device);
	if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&m->own_stream, cudaStreamNonBlocking);
	if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&m->side, cudaStreamNonBlocking);
	if (e == cudaSuccess) e = cudaEventCreateWithFlags(&m->ev_fork, cudaEventDisableTiming);
	if (e == cudaSuccess) e = cudaEventCreateWithFlags(&m->ev_join, cudaEventDisableTiming);
	if (e != cudaSuccess) { delete mm; return set_error(XALM_ERR_CUDA, "cudaStreamCreate failed: %s", cudaGetErrorString(e)); }
	m->stream = m->own_stream;
	*out = reinterpret_cast<xalm_cuda_model*>(m);
	return XALM_OK;
}

int seq_upload(SeqModel* m, const char* name, int type_id, const int* shape, int rank, const void* data, size_t nbytes) {
	if (!m || !name || !shape || !data) return set_error(XALM_ERR_INVALID, "NULL argument");
	if (m->finalized) return set_error(XALM_ERR_STATE, "upload after finalize");
	auto it = m->tensors.find(name);
	if (it == m->tensors.end()) return set_error(XALM_ERR_INVALID, "unknown tensor name '%s'", name);
	HostTensor& t = it->second;
	bool same = (size_t) rank == t.shape.size();
	size_t count = 1;
	for (int i = 0; same && i < rank; i++) same = shape[i] == t.shape[(size_t) i] || (t.shape[(size_t) i] < 0 && shape[i] > 0); // a negative extent: whatever the file has
	if (!same) return set_error(XALM_ERR_INVALID, "shape mismatch for %s", name);
	for (int i = 0; i < rank; i++) t.shape[(size_t) i] = shape[i];
	for (int dsz : t.shape) count *= (size_t) dsz;
	const size_t esz = type_id == XALM_F32 ? 4 : (type_id == XALM_F16 || type_id == XALM_BF16) ? 2 : 0;
	if (!esz) return set_error(XALM_ERR_UNSUPPORTED, "tensor %s: type %d (F32, F16 or BF16)", name, type_id);
	if (nbytes != count * esz) return set_error(XALM_ERR_INVALID, "size mismatch for %s", name);
	t.v.resize(count);
	if (type_id == XALM_F32) memcpy(t.v.data(), data, nbytes);
	else if (type_id == XALM_BF16) {
		const uint16_t* b = static_cast<const uint16_t*>(data);
		for (size_t i = 0; i < count; i++) {
			const uint32_t u = (uint32_t) b[i] << 16;
			memcpy(&t.v[i], &u, 4);
		}
	} else {
		const __half* hsrc = static_cast<const __half*>(data);
		for (size_t i = 0; i < count; i++) t.v[i] = __half2float(hsrc[i]);
	}
	t.type = type_id;
	t.got = true;
	return XALM_OK;
}

// embedding table, head matrix (absent: the embedding table serves) and final norm weight are named alike in these families
int seq_finalize(SeqModel* m) {
	if (!m) return set_error(XALM_ERR_INVALID, "model is NULL");
	if (m->finalized) return XALM_OK;
	XALM_CUDA_CHECK(cudaSetDevice(m->device));
	m->w_bf16 = m->precision != XALM_PRECISION_F32;
	for (const auto& [name, t] : m->tensors) {
		if (t.required && !t.got) return set_error(XALM_ERR_STATE, "tensor %s was not uploaded", name.c_str());
		if (t.matrix && t.got && t.type != XALM_BF16) m->w_bf16 = false; // wider checkpoints keep their precision
	}
	const int W = m->width;
	m->chunk = std::max(8, std::min(tune("seq_chunk"), 4096));
	m->keep_layers = getenv("XALM_SEQ_KEEP_LAYERS") ? atoi(getenv("XALM_SEQ_KEEP_LAYERS")) : 0;
	m->use_tc = m->w_bf16 && tune("seq_tc") > 0;
	m->tc_min_rows = std::max(1, tune("seq_tc_min"));
	XALM_TRY(upload_rows(m, {tensor_or_null(m, "embed")}, W, false, &m->embed, &m->m_head));
	if (m->tensors.count("head")) XALM_TRY(upload_rows(m, {tensor_or_null(m, "head")}, W, false, &m->w_head, &m->m_head));
	else m->w_head = m->embed; // a family that lists no head matrix multiplies by the embedding table itself
	XALM_TRY(upload_vec(m, "final.norm", &m->final_norm));
	XALM_TRY(m->hooks->finalize(m));
	if (m->use_tc) {
		XALM_TRY(tc_register(m, m->m_head, &m->t_head));
		if (m->tc_a_bytes) {
			XALM_TRY(dev_alloc(m, &m->a_hi, m->tc_a_bytes, true));
			if (tune("seq_tc") >= 2) XALM_TRY(dev_alloc(m, &m->a_lo, m->tc_a_bytes, true));
			XALM_TRY(dev_alloc(m, &m->tc_out, (size_t) m->chunk * m->tc_cols));
		} else m->use_tc = false;
		XALM_CUDA_CHECK(cudaStreamSynchronize(m->stream));
	}
	const size_t C = (size_t) m->chunk;
	XALM_TRY(dev_alloc(m, &m->logits, C * m->vocab));
	if (m->keep_layers) XALM_TRY(dev_alloc(m, &m->layer_sums, (size_t) m->n_layers * C * W, true));
	XALM_TRY(dev_alloc(m, &m->d_tokens, C));
	XALM_TRY(dev_alloc(m, &m->d_step, 1));
	XALM_CUDA_CHECK(cudaMallocHost(&m->h_logits, C * m->vocab * 4));
	for (auto& [name, t] : m->tensors) std::vector<float>().swap(t.v); // the device owns the weights from here on
	m->finalized = true;
	return XALM_OK;
}

int seq_release(SeqModel* m) {
	XALM_TRY(check_ready(m));
	XALM_CUDA_CHECK(cudaStreamSynchronize(m->stream));
	XALM_TRY(m->hooks->release(m));
	XALM_CUDA_CHECK(cudaStreamSynchronize(m->stream));
	m->pos = 0;
	m->prev_token = -1;
	return XALM_OK;
}

int seq_forward(SeqModel* m, int token, int pos, int mode, float* logits_host) {
	return seq_step(m, &token, 1, pos, mode == XALM_OUTPUT_LOGITS ? 1 : 0, logits_host, nullptr, nullptr);
}
int seq_forward_async(SeqModel* m, int token, int pos, int mode) {
	XALM_TRY(check_ready(m));
	if (pos != m->pos) return set_error(XALM_ERR_STATE, "step: position %d, but the sequence holds %d tokens", pos, m->pos);
	if (pos + 1 > m->max_tokens) return set_error(XALM_ERR_INVALID, "step: position %d exceeds max_tokens %d", pos, m->max_tokens);
	return run_pass(m, &token, 1, mode == XALM_OUTPUT_LOGITS ? 1 : 0);
}
int seq_forward_argmax(SeqModel* m, int token, int pos, int* next) {
	if (!next) return set_error(XALM_ERR_INVALID, "next_token is NULL");
	XALM_TRY(seq_step(m, &token, 1, pos, 1, nullptr, nullptr, nullptr));
	int best = 0;
	for (int i = 1; i < m->vocab; i++)
		if (m->h_logits[i] > m->h_logits[best]) best = i;
	*next = best;
	return XALM_OK;
}
int seq_sync(SeqModel* m) {
	XALM_TRY(check_ready(m));
	XALM_CUDA_CHECK(cudaStreamSynchronize(m->stream));
	return XALM_OK;
}
int seq_prefill(SeqModel* m, const int* tokens, int n, int pos0, int want, float* logits_host, const int* targets, float* probs_host) {
	return seq_step(m, tokens, n, pos0, want, logits_host, targets, probs_host);
}
int seq_prefill_async(SeqModel* m, const int* tokens, int n, int pos0, int want) {
	XALM_TRY(check_ready(m));
	if (!tokens || n <= 0) return set_error(XALM_ERR_INVALID, "step: no tokens");
	if (pos0 != m->pos) return set_error(XALM_ERR_STATE, "step: position %d, but the sequence holds %d tokens", pos0, m->pos);
	if ((long long) pos0 + n > m->max_tokens) return set_error(XALM_ERR_INVALID, "step: positions exceed max_tokens %d", m->max_tokens);
	int total = 0;
	for (int at = 0; at < n; at += m->chunk) {
		const int nc = std::min(m->chunk, n - at);
		XALM_TRY(run_pass(m, tokens + at, nc, want == 2 ? 2 : (want == 1 && at + nc == n ? 1 : 0)));
		total += m->last_launches;
	}
	m->last_launches = total;
	return XALM_OK;
}
float* seq_logits_host(SeqModel* m) { return m ? m->h_logits : nullptr; }
int seq_set_stream(SeqModel* m, void* s) {
	if (!m) return set_error(XALM_ERR_INVALID, "model is NULL");
	m->stream = s ? (cudaStream_t) s : m->own_stream;
	return XALM_OK;
}
int seq_active_bytes(SeqModel* m, long long pos, long long* bytes) {
	if (!m || !bytes) return set_error(XALM_ERR_INVALID, "NULL argument");
	// what a one-token step at `pos` reads: every weight once (one embedding row) and what the family's cache and state add
	*bytes = m->weight_bytes - (long long) (m->vocab - 1) * m->width * (m->w_bf16 ? 2 : 4) + m->hooks->active_bytes(m, pos);
	return XALM_OK;
}
int seq_last_launch_count(SeqModel* m, int* n) {
	if (!m || !n) return set_error(XALM_ERR_INVALID, "NULL argument");
	*n = m->last_launches;
	return XALM_OK;
}
// which: XALM_S_LOGITS = logits of the last pass (rows x vocab); 100 + l = the residual stream after layer l for the rows of the last
// pass (kept only when XALM_SEQ_KEEP_LAYERS=1 was set at finalize); 1000 + l = recurrent state of layer l
int seq_read_state(SeqModel* m, int which, float* dst, size_t n) {
	XALM_TRY(check_ready(m));
	if (!dst) return set_error(XALM_ERR_INVALID, "dst is NULL");
	XALM_CUDA_CHECK(cudaStreamSynchronize(m->stream));
	const float* src = nullptr;
	size_t cap = 0;
	if (which == XALM_S_LOGITS) { src = m->logits; cap = (size_t) m->chunk * m->vocab; }
	else if (which >= 100 && which < 100 + m->n_layers && m->layer_sums) {
		src = m->layer_sums + (size_t) (which - 100) * m->chunk * m->width;
		cap = (size_t) m->chunk * m->width;
	} else if (which >= 1000 && which < 1000 + m->n_layers && m->hooks->state_buffer(m, which - 1000, &src, &cap)) {
	} else return set_error(XALM_ERR_INVALID, "read_state: buffer %d", which);
	if (n > cap) return set_error(XALM_ERR_INVALID, "read_state: %zu elements requested, buffer holds %zu", n, cap);
	XALM_CUDA_CHECK(cudaMemcpy(dst, src, n * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}
int seq_expected_tensor(SeqModel* m, int index, char* name, size_t cap, int* shape4, int* rank) {
	if (!m || !name || !shape4 || !rank) return set_error(XALM_ERR_INVALID, "NULL argument");
	if (index < 0 || index >= (int) m->order.size()) return set_error(XALM_ERR_INVALID, "no tensor %d", index);
	const std::string& nm = m->order[(size_t) index];
	const HostTensor& t = m->tensors.at(nm);
	snprintf(name, cap, "%s", nm.c_str());
	*rank = (int) t.shape.size();
	for (size_t i = 0; i < t.shape.size() && i < 4; i++) shape4[i] = t.shape[i];
	return XALM_OK;
}
int seq_info(SeqModel* m, const char* key, long long* value) {
	if (!m || !key || !value) return set_error(XALM_ERR_INVALID, "NULL argument");
	const std::string k = key;
	if (k == "vocab_size") *value = m->vocab;
	else if (k == "dim") *value = m->width;
	else if (k == "n_layers") *value = m->n_layers;
	else if (k == "max_tokens") *value = m->max_tokens;
	else if (k == "position") *value = m->pos;
	else if (k == "chunk") *value = m->chunk;
	else return set_error(XALM_ERR_INVALID, "unknown property '%s'", key);
	return XALM_OK;
}

// the family table speaks in opaque handles
template <auto F>
struct Thunk;
template <typename... A, int (*F)(SeqModel*, A...)>
struct Thunk<F> {
	static int call(xalm_cuda_model* h, A... a) { return F(reinterpret_cast<SeqModel*>(h), a...); }
};
void seq_destroy_thunk(xalm_cuda_model* h) { seq_destroy(reinterpret_cast<SeqModel*>(h)); }
float* seq_logits_thunk(xalm_cuda_model* h) { return seq_logits_host(reinterpret_cast<SeqModel*>(h)); }

// the table of a family named `name` whose handles `create` makes (seq_create<its model>)
ModelFamily seq_family_table(const char* name, int (*create)(const char*, int, int, int, xalm_cuda_model**)) {
	return ModelFamily{name, create, Thunk<seq_upload>::call, nullptr, nullptr, Thunk<seq_finalize>::call, seq_destroy_thunk, nullptr, nullptr, nullptr,
	                   Thunk<seq_set_stream>::call, Thunk<seq_forward>::call, Thunk<seq_forward_argmax>::call, Thunk<seq_forward_async>::call,
	                   Thunk<seq_sync>::call, Thunk<seq_prefill>::call, Thunk<seq_prefill_async>::call, seq_logits_thunk, Thunk<seq_active_bytes>::call,
	                   Thunk<seq_last_launch_count>::call, Thunk<seq_read_state>::call, nullptr, nullptr, Thunk<seq_release>::call,
	                   Thunk<seq_expected_tensor>::call, Thunk<seq_info>::call, nullptr};
}

} // namespace
} // namespace seq
} // namespace xalm
