// mix_ops.cu — op-level entry points for the mechanisms of mix_ops.cuh (include/xalm_cuda.h, "mechanism ops"): host arrays in,
// host arrays out, one kernel family each, so that a test can hold every mechanism against a plain fp32 restatement without
// building a model around it.  They launch the SAME kernels the config.json families run.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <vector>

#define XALM_SECONDARY_TU
#include "common.cuh"
#include "family.h"
#include "mix_ops.cuh"
#include "delta_ops.cuh"
#include "conv_ops.cuh"
#include "latent_ops.cuh"
#include "moe_ops.cuh"

using namespace xalm;
using namespace xalm::mix;

namespace {

// device buffers of one call, freed when it returns
struct Pool {
	std::vector<void*> p;
	~Pool() {
		for (void* q : p) cudaFree(q);
	}
	template <typename T>
	T* put(const T* host, size_t n) { // NULL stays NULL
		if (!host) return nullptr;
		T* d = raw<T>(n);
		if (d && cudaMemcpy(d, host, n * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess) return nullptr;
		return d;
	}
	template <typename T>
	T* raw(size_t n) {
		void* d = nullptr;
		if (cudaMalloc(&d, std::max<size_t>(n * sizeof(T), 16)) != cudaSuccess) return nullptr;
		p.push_back(d);
		cudaMemset(d, 0, std::max<size_t>(n * sizeof(T), 16));
		return static_cast<T*>(d);
	}
};

int finish(const char* what) {
	cudaError_t e = cudaGetLastError();
	if (e == cudaSuccess) e = cudaDeviceSynchronize();
	if (e != cudaSuccess) return set_error(XALM_ERR_CUDA, "%s failed: %s", what, cudaGetErrorString(e));
	return XALM_OK;
}

uint16_t bf16_bits(float f) {
	const __nv_bfloat16 b = __float2bfloat16_rn(f);
	uint16_t u;
	memcpy(&u, &b, 2);
	return u;
}

} // namespace

static int swa_attention_op(float* out, const float* q, const float* gate, const float* k, const float* v, int T, int pos0, int H, int G, int d, int dv,
                            int window, int keep_first, float scale, float softcap, const float* r1, const float* r2, const float* talk, int ring, int n_splits,
                            int cache_bf16, const float* sink = nullptr, float out_scale = 0.f) {
	if (!out || !q || !k || !v || T <= 0 || pos0 < 0 || H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0 || window <= 0 || n_splits < 1 || keep_first < 0)
		return set_error(XALM_ERR_INVALID, "swa_attention: bad argument");
	const int n = pos0 + T;
	const long long need = std::min<long long>(std::max(1, n - keep_first), (long long) window - 1 + T);
	if (ring < need) return set_error(XALM_ERR_INVALID, "swa_attention: a ring of %d slots cannot hold %lld live positions", ring, need);
	if (!r1 != !r2) return set_error(XALM_ERR_INVALID, "swa_attention: r1 and r2 come together");
	const size_t smem = swa_smem_bytes(H, d, dv);
	if (!swa_pick_tq(H, G, d, dv, T) && smem > 200 * 1024) return set_error(XALM_ERR_UNSUPPORTED, "swa_attention: heads need %zu bytes of shared memory", smem);
	Pool pool;
	// the ring as the cache manager leaves it: position p lives in slot p % ring, older positions are overwritten
	const size_t esz = cache_bf16 ? 2 : 4;
	const int slots = keep_first + ring; // the first keep_first positions have slots of their own
	std::vector<uint8_t> kr((size_t) slots * G * d * esz, 0), vr((size_t) slots * G * dv * esz, 0);
	for (int p = 0; p < n; p++) {
		const int slot = p < keep_first ? p : keep_first + (p - keep_first) % ring;
		for (int c = 0; c < G * d; c++) {
			const float x = k[(size_t) p * G * d + c];
			if (cache_bf16) reinterpret_cast<uint16_t*>(kr.data())[(size_t) slot * G * d + c] = bf16_bits(x);
			else reinterpret_cast<float*>(kr.data())[(size_t) slot * G * d + c] = x;
		}
		for (int c = 0; c < G * dv; c++) {
			const float x = v[(size_t) p * G * dv + c];
			if (cache_bf16) reinterpret_cast<uint16_t*>(vr.data())[(size_t) slot * G * dv + c] = bf16_bits(x);
			else reinterpret_cast<float*>(vr.data())[(size_t) slot * G * dv + c] = x;
		}
	}
	const SeqStep st = {pos0, T};
	SwaArgs a = {};
	a.q = pool.put(q, (size_t) T * H * d);
	a.gate = pool.put(gate, (size_t) T * H * dv);
	a.ldq = H * d; a.q_off = 0; a.g_off = 0;
	a.ldg = H * dv;
	a.kc = pool.put(kr.data(), kr.size());
	a.vc = pool.put(vr.data(), vr.size());
	a.ring = ring; a.keep_first = keep_first; a.H = H; a.G = G; a.d = d; a.dv = dv; a.window = window; a.scale = scale; a.softcap = softcap;
	a.r1 = pool.put(r1, (size_t) H); a.r2 = pool.put(r2, (size_t) H); a.talk = pool.put(talk, (size_t) H * H);
	a.step = pool.put(&st, 1);
	a.sink = pool.put(sink, (size_t) H); a.out_scale = out_scale;
	float* d_out = pool.raw<float>((size_t) T * H * dv);
	a.out = d_out;
	a.n_splits = n_splits;
	a.part_cap = T * n_splits;
	a.part_o = pool.raw<float>((size_t) T * n_splits * H * dv);
	a.part_ml = pool.raw<float>((size_t) T * n_splits * H * 2);
	if (!a.q || !a.kc || !a.vc || !a.step || !d_out || !a.part_o || !a.part_ml) return set_error(XALM_ERR_CUDA, "swa_attention: device allocation failed");
	XALM_TRY(launch_swa(a, T, cache_bf16 == 0, nullptr));
	XALM_TRY(finish("swa_attention"));
	XALM_CUDA_CHECK(cudaMemcpy(out, d_out, (size_t) T * H * dv * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}

extern "C" {

int xalm_cuda_swa_attention(float* out, const float* q, const float* gate, const float* k, const float* v, int T, int pos0, int H, int G, int d, int dv,
                            int window, float scale, float softcap, const float* r1, const float* r2, const float* talk, int ring, int n_splits,
                            int cache_bf16) {
	return swa_attention_op(out, q, gate, k, v, T, pos0, H, G, d, dv, window, 0, scale, softcap, r1, r2, talk, ring, n_splits, cache_bf16);
}
int xalm_cuda_swa_attention_kept(float* out, const float* q, const float* k, const float* v, int T, int pos0, int H, int G, int d, int dv, int window,
                                 int keep_first, float scale, int ring, int n_splits, int cache_bf16) {
	return swa_attention_op(out, q, nullptr, k, v, T, pos0, H, G, d, dv, window, keep_first, scale, 0.f, nullptr, nullptr, nullptr, ring, n_splits, cache_bf16);
}

int xalm_cuda_hgrn2(float* out, float* state, const float* qz, const float* fz, const float* v, int T, int H, int d, int dv, const float* f_bias,
                    const float* lower, const float* norm_w, float eps) {
	if (!out || !state || !qz || !fz || !v || T <= 0 || H <= 0 || d <= 0 || dv <= 0) return set_error(XALM_ERR_INVALID, "hgrn2: bad argument");
	const size_t smem = hgrn2_smem_bytes(d, dv);
	if (!hgrn2_cols_ok(d, dv, T) && (smem > 200 * 1024 || dv > 1024)) return set_error(XALM_ERR_UNSUPPORTED, "hgrn2: a head's state needs %zu bytes of shared memory", smem);
	Pool pool;
	const int ld = 2 * H * d + H * dv;
	std::vector<float> proj((size_t) T * ld);
	for (int t = 0; t < T; t++) {
		memcpy(&proj[(size_t) t * ld], qz + (size_t) t * H * d, (size_t) H * d * 4);
		memcpy(&proj[(size_t) t * ld + H * d], fz + (size_t) t * H * d, (size_t) H * d * 4);
		memcpy(&proj[(size_t) t * ld + 2 * H * d], v + (size_t) t * H * dv, (size_t) H * dv * 4);
	}
	const SeqStep st = {0, T};
	Hgrn2Args a = {};
	a.proj = pool.put(proj.data(), proj.size());
	a.ld = ld; a.q_off = 0; a.f_off = H * d; a.v_off = 2 * H * d;
	a.H = H; a.d = d; a.dv = dv;
	a.f_bias = pool.put(f_bias, (size_t) H * d); a.lower = pool.put(lower, (size_t) H * d); a.norm_w = pool.put(norm_w, (size_t) dv);
	a.eps = eps;
	a.state = pool.put(state, (size_t) H * d * dv);
	a.step = pool.put(&st, 1);
	float* d_out = pool.raw<float>((size_t) T * H * dv);
	a.out = d_out;
	a.max_rows = T;
	if (!a.proj || !a.state || !a.step || !d_out) return set_error(XALM_ERR_CUDA, "hgrn2: device allocation failed");
	XALM_TRY(launch_hgrn2(a, nullptr));
	XALM_TRY(finish("hgrn2"));
	XALM_CUDA_CHECK(cudaMemcpy(out, d_out, (size_t) T * H * dv * 4, cudaMemcpyDeviceToHost));
	XALM_CUDA_CHECK(cudaMemcpy(state, a.state, (size_t) H * d * dv * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}

int xalm_cuda_hyper_norm(float* h, const float* xs, int S, int T, int W, const float* a, const float* w, int one_plus, float eps) {
	if (!h || !xs || !w || S < 1 || S > MAX_STREAMS || T <= 0 || W <= 0) return set_error(XALM_ERR_INVALID, "hyper_norm: bad argument");
	Pool pool;
	const float* d_xs = pool.put(xs, (size_t) S * T * W);
	const float* d_a = pool.put(a, (size_t) S);
	const float* d_w = pool.put(w, (size_t) W);
	float* d_h = pool.raw<float>((size_t) T * W);
	if (!d_xs || !d_w || !d_h) return set_error(XALM_ERR_CUDA, "hyper_norm: device allocation failed");
	XALM_TRY(launch_hc_norm(d_xs, S, (size_t) T * W, d_a, d_w, one_plus, eps, W, d_h, nullptr, T, nullptr));
	XALM_TRY(finish("hyper_norm"));
	XALM_CUDA_CHECK(cudaMemcpy(h, d_h, (size_t) T * W * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}

int xalm_cuda_dual_norm_hyper(float* xs, const float* a, const float* b, const float* wa, const float* wb, float eps, int S, int T, int W,
                              const float* mix, const float* out_coef, const float* scale) {
	if (!xs || !a || !b || !wa || !wb || S < 1 || S > MAX_STREAMS || T <= 0 || W <= 0) return set_error(XALM_ERR_INVALID, "dual_norm_hyper: bad argument");
	Pool pool;
	RowsEpi e;
	e.kind = EPI_HC;
	e.xs = pool.put(xs, (size_t) S * T * W);
	e.S = S;
	e.stream_stride = (size_t) T * W;
	e.hmix = pool.put(mix, (size_t) S * S);
	e.hout = pool.put(out_coef, (size_t) S);
	e.scale = pool.put(scale, (size_t) W);
	const float *d_a = pool.put(a, (size_t) T * W), *d_b = pool.put(b, (size_t) T * W), *d_wa = pool.put(wa, (size_t) W), *d_wb = pool.put(wb, (size_t) W);
	if (!e.xs || !d_a || !d_b || !d_wa || !d_wb) return set_error(XALM_ERR_CUDA, "dual_norm_hyper: device allocation failed");
	XALM_TRY(launch_dual_norm_hc(d_a, d_b, d_wa, d_wb, eps, W, e, T, 0));
	XALM_TRY(finish("dual_norm_hyper"));
	XALM_CUDA_CHECK(cudaMemcpy(xs, e.xs, (size_t) S * T * W * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}

int xalm_cuda_glu_rows(float* out, const float* x, const float* w_gate, const float* w_up, int T, int ff, int K, float limit, float alpha, int w_bf16) {
	if (!out || !x || !w_gate || !w_up || T <= 0 || ff <= 0 || K <= 0) return set_error(XALM_ERR_INVALID, "glu_rows: bad argument");
	Pool pool;
	// gate and up rows interleaved, as the families store them
	std::vector<float> wf((size_t) 2 * ff * K);
	for (int i = 0; i < ff; i++) {
		memcpy(&wf[(size_t) (2 * i) * K], w_gate + (size_t) i * K, (size_t) K * 4);
		memcpy(&wf[(size_t) (2 * i + 1) * K], w_up + (size_t) i * K, (size_t) K * 4);
	}
	void* d_w;
	if (w_bf16) {
		std::vector<uint16_t> wb(wf.size());
		for (size_t i = 0; i < wf.size(); i++) wb[i] = bf16_bits(wf[i]);
		d_w = pool.put(wb.data(), wb.size());
	} else d_w = pool.put(wf.data(), wf.size());
	const float* d_x = pool.put(x, (size_t) T * K);
	RowsEpi e;
	e.kind = EPI_GLU;
	e.out = pool.raw<float>((size_t) T * ff);
	e.ldo = ff;
	e.limit = limit;
	e.alpha = alpha;
	if (!d_w || !d_x || !e.out) return set_error(XALM_ERR_CUDA, "glu_rows: device allocation failed");
	XALM_TRY(launch_rows(d_x, K, d_w, w_bf16 != 0, T, 2 * ff, K, e, nullptr));
	XALM_TRY(finish("glu_rows"));
	XALM_CUDA_CHECK(cudaMemcpy(out, e.out, (size_t) T * ff * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}

int xalm_cuda_group_norm_residual(float* x_out, float* avg_out, const float* y, int parts, const float* part_w, const float* w, int groups, float eps,
                                  const float* x_in, const float* hist, int n_hist, const float* dwa, int T, int W) {
	if (!x_out || !y || !w || parts < 1 || groups < 1 || T <= 0 || W <= 0 || W % groups || (dwa && (!avg_out || (n_hist > 0 && !hist))))
		return set_error(XALM_ERR_INVALID, "group_norm_residual: bad argument");
	Pool pool;
	GroupNormArgs g;
	g.y = pool.put(y, (size_t) T * parts * W); g.ldy = W; g.parts = parts;
	g.part_w = pool.put(part_w, (size_t) T * parts);
	g.w = pool.put(w, (size_t) W); g.groups = groups; g.width = W; g.eps = eps;
	g.x_in = pool.put(x_in, (size_t) T * W);
	g.x_out = pool.raw<float>((size_t) T * W);
	g.hist = pool.put(hist, (size_t) std::max(1, n_hist) * T * W); g.hist_stride = (size_t) T * W; g.n_hist = n_hist;
	g.dwa = pool.put(dwa, (size_t) n_hist + 1);
	g.avg_out = dwa ? pool.raw<float>((size_t) T * W) : nullptr;
	if (!g.y || !g.w || !g.x_out) return set_error(XALM_ERR_CUDA, "group_norm_residual: device allocation failed");
	XALM_TRY(group_norm_prepare(W, groups));
	XALM_TRY(launch_group_norm(g, T, nullptr));
	XALM_TRY(finish("group_norm_residual"));
	XALM_CUDA_CHECK(cudaMemcpy(x_out, g.x_out, (size_t) T * W * 4, cudaMemcpyDeviceToHost));
	if (dwa) XALM_CUDA_CHECK(cudaMemcpy(avg_out, g.avg_out, (size_t) T * W * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}

static int qkv_post_op(float* q_out, float* k_out, float* v_out, const float* proj, int T, int pos0, int H, int G, int d, int dv, const float* bq,
                       const float* bk, const float* bv, const float* freq, int rot_half, int norm_qk, int norm_v, float eps, int keep_first, int ring,
                       float rot_mag, int v_from_k) {
	if (!q_out || !k_out || !v_out || !proj || T <= 0 || pos0 < 0 || H <= 0 || G <= 0 || d <= 0 || dv <= 0 || 2 * rot_half > d || keep_first < 0 || ring < 1)
		return set_error(XALM_ERR_INVALID, "qkv_post: bad argument");
	Pool pool;
	if (v_from_k && dv != d) return set_error(XALM_ERR_INVALID, "qkv_post: values that are the keys have the keys' size");
	const int ld = H * d + G * d + (v_from_k ? 0 : G * dv), slots = keep_first + ring;
	const SeqStep st = {pos0, T};
	QkvPostArgs a = {};
	a.proj = pool.put(proj, (size_t) T * ld); a.ld = ld; a.q_off = 0; a.k_off = H * d; a.v_off = v_from_k ? H * d : H * d + G * d;
	a.rot_mag = rot_mag;
	a.H = H; a.G = G; a.d = d; a.dv = dv;
	a.bq = pool.put(bq, (size_t) H * d); a.bk = pool.put(bk, (size_t) G * d); a.bv = pool.put(bv, (size_t) G * dv);
	a.freq = rot_half ? pool.put(freq, (size_t) rot_half) : nullptr; a.rot_half = rot_half;
	a.norm_qk = norm_qk; a.norm_v = norm_v; a.eps = eps;
	float* kc = pool.raw<float>((size_t) slots * G * d);
	float* vc = pool.raw<float>((size_t) slots * G * dv);
	a.kc = kc; a.vc = vc; a.cache_f32 = 1; a.keep_first = keep_first; a.ring = ring;
	a.step = pool.put(&st, 1);
	if (!a.proj || !kc || !vc || !a.step) return set_error(XALM_ERR_CUDA, "qkv_post: device allocation failed");
	XALM_TRY(launch_qkv_post(a, T, nullptr));
	XALM_TRY(finish("qkv_post"));
	std::vector<float> back((size_t) T * ld);
	XALM_CUDA_CHECK(cudaMemcpy(back.data(), a.proj, back.size() * 4, cudaMemcpyDeviceToHost));
	for (int t = 0; t < T; t++) memcpy(q_out + (size_t) t * H * d, &back[(size_t) t * ld], (size_t) H * d * 4);
	// the whole cache, slot by slot, so that a test sees where each position went
	XALM_CUDA_CHECK(cudaMemcpy(k_out, kc, (size_t) slots * G * d * 4, cudaMemcpyDeviceToHost));
	XALM_CUDA_CHECK(cudaMemcpy(v_out, vc, (size_t) slots * G * dv * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}

int xalm_cuda_qkv_post(float* q_out, float* k_out, float* v_out, const float* proj, int T, int pos0, int H, int G, int d, int dv, const float* bq,
                       const float* bk, const float* bv, const float* freq, int rot_half, int norm_qk, int norm_v, float eps, int keep_first, int ring) {
	return qkv_post_op(q_out, k_out, v_out, proj, T, pos0, H, G, d, dv, bq, bk, bv, freq, rot_half, norm_qk, norm_v, eps, keep_first, ring, 0.f, 0);
}
int xalm_cuda_qk_post(float* q_out, float* k_out, float* v_out, const float* proj, int T, int pos0, int H, int G, int d, const float* freq, int rot_half,
                      float rot_mag, int ring) {
	return qkv_post_op(q_out, k_out, v_out, proj, T, pos0, H, G, d, d, nullptr, nullptr, nullptr, freq, rot_half, 0, 0, 0.f, 0, ring, rot_mag, 1);
}

int xalm_cuda_delta_rule(float* out, float* state, float* conv_state, const float* q, const float* k, const float* v, const float* gate, const float* b,
                         const float* a_in, int T, int H, int G, int d, int dv, int taps, const float* wq, const float* wk, const float* wv,
                         const float* A_log, const float* dt_bias, const float* norm_w, float eps, float unit_eps, float q_scale) {
	if (!out || !state || !conv_state || !q || !k || !v || !gate || !b || !a_in || !wq || !wk || !wv || !A_log || !dt_bias || T <= 0 || H <= 0 || G <= 0 || H % G ||
	    d <= 0 || dv <= 0 || taps < 1)
		return set_error(XALM_ERR_INVALID, "delta_rule: bad argument");
	if (!delta_ok(d, dv)) return set_error(XALM_ERR_UNSUPPORTED, "delta_rule: a state of %d x %d per head", d, dv);
	Pool pool;
	const int nq = G * d, nv = H * dv, Cc = 2 * nq + nv, ld = Cc + nv + 2 * H;
	std::vector<float> proj((size_t) T * ld);
	for (int t = 0; t < T; t++) {
		float* row = &proj[(size_t) t * ld];
		memcpy(row, q + (size_t) t * nq, (size_t) nq * 4);
		memcpy(row + nq, k + (size_t) t * nq, (size_t) nq * 4);
		memcpy(row + 2 * nq, v + (size_t) t * nv, (size_t) nv * 4);
		memcpy(row + Cc, gate + (size_t) t * nv, (size_t) nv * 4);
		memcpy(row + Cc + nv, b + (size_t) t * H, (size_t) H * 4);
		memcpy(row + Cc + nv + H, a_in + (size_t) t * H, (size_t) H * 4);
	}
	const SeqStep st = {0, T};
	DeltaArgs a = {};
	a.proj = pool.put(proj.data(), proj.size()); a.ld = ld;
	a.q_off = 0; a.k_off = nq; a.v_off = 2 * nq; a.g_off = Cc; a.b_off = Cc + nv; a.a_off = Cc + nv + H;
	a.H = H; a.G = G; a.d = d; a.dv = dv; a.taps = taps;
	a.wq = pool.put(wq, (size_t) nq * taps); a.wk = pool.put(wk, (size_t) nq * taps); a.wv = pool.put(wv, (size_t) nv * taps);
	a.A_log = pool.put(A_log, (size_t) H); a.dt_bias = pool.put(dt_bias, (size_t) H); a.norm_w = pool.put(norm_w, (size_t) dv);
	a.eps = eps; a.unit_eps = unit_eps; a.q_scale = q_scale;
	const size_t ncs = (size_t) std::max(1, taps - 1) * Cc;
	a.conv_state = pool.put(conv_state, ncs);
	a.state = pool.put(state, (size_t) H * d * dv);
	a.ldp = Cc + 2 * H;
	a.prep = pool.raw<float>((size_t) T * a.ldp);
	a.out = pool.raw<float>((size_t) T * nv);
	a.step = pool.put(&st, 1);
	if (!a.proj || !a.conv_state || !a.state || !a.prep || !a.out || !a.step) return set_error(XALM_ERR_CUDA, "delta_rule: device allocation failed");
	XALM_TRY(delta_prepare(d, dv));
	XALM_TRY(launch_delta(a, T, nullptr));
	XALM_TRY(finish("delta_rule"));
	XALM_CUDA_CHECK(cudaMemcpy(out, a.out, (size_t) T * nv * 4, cudaMemcpyDeviceToHost));
	XALM_CUDA_CHECK(cudaMemcpy(state, a.state, (size_t) H * d * dv * 4, cudaMemcpyDeviceToHost));
	if (taps > 1) XALM_CUDA_CHECK(cudaMemcpy(conv_state, a.conv_state, ncs * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}

} // extern "C"

static int moe_ffn_op(float* out_pairs, int* idx, float* wgt, const float* h, const float* w_router, const float* w_gate, const float* w_up,
                      const float* w_down, int T, int K, int E, int top, int ff, int n_groups, int keep_groups, int act, int w_bf16, int score_kind,
                      int group_kind, int renormalise, float limit, float* x_io) {
	if (!out_pairs || !idx || !wgt || !h || !w_router || !w_gate || !w_up || !w_down || T <= 0 || K <= 0 || E <= 0 || top <= 0 || ff <= 0)
		return set_error(XALM_ERR_INVALID, "moe_ffn: bad argument");
	Pool pool;
	// gate and up rows interleaved expert after expert, as the families store them
	std::vector<float> gu((size_t) E * 2 * ff * K);
	for (int e = 0; e < E; e++)
		for (int i = 0; i < ff; i++) {
			memcpy(&gu[((size_t) e * 2 * ff + 2 * i) * K], w_gate + ((size_t) e * ff + i) * K, (size_t) K * 4);
			memcpy(&gu[((size_t) e * 2 * ff + 2 * i + 1) * K], w_up + ((size_t) e * ff + i) * K, (size_t) K * 4);
		}
	auto put_w = [&](const float* src, size_t n) -> void* {
		if (!w_bf16) return pool.put(src, n);
		std::vector<uint16_t> wb(n);
		for (size_t i = 0; i < n; i++) wb[i] = bf16_bits(src[i]);
		return pool.put(wb.data(), n);
	};
	const SeqStep st = {0, T};
	const SeqStep* d_st = pool.put(&st, 1);
	const int P = T * top, max_tiles = moe_max_tiles(P, E);
	MoeRouteArgs ra = {};
	ra.h = pool.put(h, (size_t) T * K); ra.ldh = K; ra.w = put_w(w_router, (size_t) E * K); ra.w_bf16 = w_bf16;
	ra.E = E; ra.top = top; ra.K = K; ra.n_groups = n_groups; ra.keep_groups = keep_groups;
	ra.idx = pool.raw<int>((size_t) P); ra.wgt = pool.raw<float>((size_t) P); ra.step = d_st;
	ra.score_kind = score_kind; ra.group_kind = group_kind; ra.renormalise = renormalise; ra.renorm_eps = 1e-20f;
	MoeSortArgs so = {ra.idx, top, E, d_st, pool.raw<int>((size_t) P), pool.raw<int>((size_t) 3 * max_tiles), pool.raw<int>(1), nullptr, nullptr};
	MoeGemmArgs ga = {};
	ga.A = ra.h; ga.lda = K; ga.a_div = top; ga.W = put_w(gu.data(), gu.size()); ga.N = 2 * ff; ga.K = K;
	ga.sorted = so.sorted; ga.tiles = so.tiles; ga.n_tiles = so.n_tiles;
	ga.idx = ra.idx; ga.step = d_st; ga.top = top;
	float* hid = pool.raw<float>((size_t) P * ff);
	float* outp = pool.raw<float>((size_t) P * K);
	ga.e.kind = EPI_GLU; ga.e.glu_act = act; ga.e.out = hid; ga.e.ldo = ff; ga.e.limit = limit;
	void* d_down = put_w(w_down, (size_t) E * K * ff);
	if (!d_st || !ra.h || !ra.w || !ra.idx || !ra.wgt || !so.sorted || !so.tiles || !so.n_tiles || !ga.W || !hid || !outp || !d_down)
		return set_error(XALM_ERR_CUDA, "moe_ffn: device allocation failed");
	XALM_TRY(moe_prepare(K, E, n_groups));
	XALM_TRY(launch_moe_router(ra, T, nullptr));
	XALM_TRY(launch_moe_sort(so, nullptr));
	XALM_TRY(launch_moe_gemm(ga, w_bf16 != 0, P, E, nullptr));
	ga.A = hid; ga.lda = ff; ga.a_div = 1; ga.W = d_down; ga.N = K; ga.K = ff;
	ga.e = RowsEpi();
	ga.e.kind = EPI_STORE; ga.e.out = outp; ga.e.ldo = K;
	XALM_TRY(launch_moe_gemm(ga, w_bf16 != 0, P, E, nullptr));
	float* d_x = pool.put(x_io, (size_t) T * K);
	if (x_io) { // the residual stream takes the weighted sum of each token's rows
		if (!d_x) return set_error(XALM_ERR_CUDA, "moe_ffn: device allocation failed");
		MoeCombineArgs ca = {outp, K, top, K, ra.wgt, nullptr, d_x, d_x, d_st};
		XALM_TRY(launch_moe_combine(ca, T, nullptr));
	}
	XALM_TRY(finish("moe_ffn"));
	if (x_io) XALM_CUDA_CHECK(cudaMemcpy(x_io, d_x, (size_t) T * K * 4, cudaMemcpyDeviceToHost));
	XALM_CUDA_CHECK(cudaMemcpy(out_pairs, outp, (size_t) P * K * 4, cudaMemcpyDeviceToHost));
	XALM_CUDA_CHECK(cudaMemcpy(idx, ra.idx, (size_t) P * 4, cudaMemcpyDeviceToHost));
	XALM_CUDA_CHECK(cudaMemcpy(wgt, ra.wgt, (size_t) P * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}

extern "C" {

int xalm_cuda_moe_ffn(float* out_pairs, int* idx, float* wgt, const float* h, const float* w_router, const float* w_gate, const float* w_up,
                      const float* w_down, int T, int K, int E, int top, int ff, int n_groups, int keep_groups, int act, int w_bf16) {
	return moe_ffn_op(out_pairs, idx, wgt, h, w_router, w_gate, w_up, w_down, T, K, E, top, ff, n_groups, keep_groups, act, w_bf16, MOE_SCORE_SIGMOID,
	                  MOE_GROUP_TOP2_SUM, 0, INFINITY, nullptr);
}
int xalm_cuda_moe_ffn_routed(float* out_pairs, int* idx, float* wgt, float* x_io, const float* h, const float* w_router, const float* w_gate,
                             const float* w_up, const float* w_down, int T, int K, int E, int top, int ff, int n_groups, int keep_groups, int act,
                             int w_bf16, int score_kind, int group_kind, int renormalise, float limit) {
	return moe_ffn_op(out_pairs, idx, wgt, h, w_router, w_gate, w_up, w_down, T, K, E, top, ff, n_groups, keep_groups, act, w_bf16, score_kind, group_kind,
	                  renormalise, limit, x_io);
}

int xalm_cuda_retention(float* out, float* state, const float* q, const float* k, const float* v, const float* gate, int T, int pos0, int H, int d, int dv,
                        const float* decay, const float* freq, int rot_half, float k_scale, float eps) {
	if (!out || !state || !q || !k || !v || !decay || T <= 0 || pos0 < 0 || H <= 0 || d <= 0 || dv <= 0 || rot_half < 0 || 2 * rot_half > d || (rot_half && !freq))
		return set_error(XALM_ERR_INVALID, "retention: bad argument");
	const size_t smem = hgrn2_smem_bytes(d, dv);
	if (!hgrn2_cols_ok(d, dv, T) && (smem > 200 * 1024 || dv > 1024)) return set_error(XALM_ERR_UNSUPPORTED, "retention: a head's state needs %zu bytes of shared memory", smem);
	Pool pool;
	const int ld = 2 * H * d + 2 * H * dv; // q | k | v | gate, as the family's input projection leaves them
	std::vector<float> proj((size_t) T * ld, 0.f);
	for (int t = 0; t < T; t++) {
		memcpy(&proj[(size_t) t * ld], q + (size_t) t * H * d, (size_t) H * d * 4);
		memcpy(&proj[(size_t) t * ld + H * d], k + (size_t) t * H * d, (size_t) H * d * 4);
		memcpy(&proj[(size_t) t * ld + 2 * H * d], v + (size_t) t * H * dv, (size_t) H * dv * 4);
		if (gate) memcpy(&proj[(size_t) t * ld + 2 * H * d + H * dv], gate + (size_t) t * H * dv, (size_t) H * dv * 4);
	}
	const SeqStep st = {pos0, T};
	float* d_proj = pool.put(proj.data(), proj.size());
	const SeqStep* d_st = pool.put(&st, 1);
	const float* d_freq = pool.put(freq, (size_t) rot_half);
	Hgrn2Args a = {};
	a.proj = d_proj; a.ld = ld; a.q_off = 0; a.k_off = H * d; a.v_off = 2 * H * d;
	a.H = H; a.d = d; a.dv = dv;
	a.decay = pool.put(decay, (size_t) H); a.k_scale = k_scale; a.norm_plain = 1; a.eps = eps;
	if (gate) { a.gate = d_proj; a.ldg = ld; a.g_off = 2 * H * d + H * dv; }
	a.state = pool.put(state, (size_t) H * d * dv);
	a.step = d_st;
	a.out = pool.raw<float>((size_t) T * H * dv);
	a.max_rows = T;
	if (!d_proj || !d_st || !a.decay || !a.state || !a.out || (rot_half && !d_freq)) return set_error(XALM_ERR_CUDA, "retention: device allocation failed");
	if (rot_half) {
		RopeHeadsArgs ra = {};
		ra.src = d_proj; ra.dst = d_proj; ra.lds = ra.ldd = ld; ra.src_stride = ra.dst_stride = d;
		ra.heads = 2 * H; ra.n = d; ra.rot_half = rot_half; ra.freq = d_freq; ra.step = d_st;
		XALM_TRY(launch_rope_heads(ra, T, nullptr));
	}
	XALM_TRY(hgrn2_prepare(d, dv));
	XALM_TRY(launch_hgrn2(a, nullptr));
	XALM_TRY(finish("retention"));
	XALM_CUDA_CHECK(cudaMemcpy(out, a.out, (size_t) T * H * dv * 4, cudaMemcpyDeviceToHost));
	XALM_CUDA_CHECK(cudaMemcpy(state, a.state, (size_t) H * d * dv * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}

int xalm_cuda_latent_post(float* cq_out, float* cache_out, const float* proj, int T, int pos0, int q_rank, int kv_rank, int rot, const float* q_norm,
                          const float* kv_norm, const float* freq, float eps, int ring, int cache_bf16) {
	if (!proj || T <= 0 || pos0 < 0 || q_rank < 0 || kv_rank < 0 || rot < 0 || rot % 2 || ring <= 0 || (q_rank && (!cq_out || !q_norm)) ||
	    (kv_rank && (!cache_out || !kv_norm)) || (rot && !freq))
		return set_error(XALM_ERR_INVALID, "latent_post: bad argument");
	Pool pool;
	const int ld = q_rank + kv_rank + rot, cl = kv_rank + rot;
	const SeqStep st = {pos0, T};
	LatentPostArgs a = {};
	a.proj = pool.put(proj, (size_t) T * ld); a.ld = ld;
	a.q_off = 0; a.q_rank = q_rank; a.q_norm = pool.put(q_norm, (size_t) q_rank); a.cq = pool.raw<float>((size_t) T * std::max(1, q_rank)); a.ldc = q_rank;
	a.kv_off = q_rank; a.kv_rank = kv_rank; a.rot = kv_rank ? rot : 0; a.kv_norm = pool.put(kv_norm, (size_t) kv_rank); a.freq = pool.put(freq, (size_t) rot / 2);
	a.eps = eps; a.cache_f32 = !cache_bf16; a.ring = ring;
	a.cache = pool.raw<float>((size_t) ring * std::max(1, cl));
	a.step = pool.put(&st, 1);
	if (!a.proj || !a.cq || !a.cache || !a.step) return set_error(XALM_ERR_CUDA, "latent_post: device allocation failed");
	XALM_TRY(launch_latent_post(a, T, nullptr));
	XALM_TRY(finish("latent_post"));
	if (q_rank) XALM_CUDA_CHECK(cudaMemcpy(cq_out, a.cq, (size_t) T * q_rank * 4, cudaMemcpyDeviceToHost));
	if (kv_rank) {
		if (!cache_bf16) XALM_CUDA_CHECK(cudaMemcpy(cache_out, a.cache, (size_t) ring * cl * 4, cudaMemcpyDeviceToHost));
		else {
			std::vector<uint16_t> hb((size_t) ring * cl);
			XALM_CUDA_CHECK(cudaMemcpy(hb.data(), a.cache, hb.size() * 2, cudaMemcpyDeviceToHost));
			for (size_t i = 0; i < hb.size(); i++) {
				const uint32_t u = (uint32_t) hb[i] << 16;
				memcpy(&cache_out[i], &u, 4);
			}
		}
	}
	return XALM_OK;
}

int xalm_cuda_latent_attend(float* out, const float* q, const float* cache, const float* gate, int T, int pos0, int H, int d, int r, int dv, int R, int ld,
                            const float* uk, const float* uv, const float* freq, float scale, int n_splits, int cache_bf16, int w_bf16) {
	if (!out || !q || !cache || !uk || !uv || T <= 0 || pos0 < 0 || H <= 0 || d <= 0 || r < 0 || r % 2 || dv <= 0 || R <= 0 || ld < R + r || n_splits < 0 || (r && !freq))
		return set_error(XALM_ERR_INVALID, "latent_attend: bad argument");
	const int n = pos0 + T, da = R + r;
	if (!swa_pick_tq(H, 1, da, R, T) && swa_smem_bytes(H, da, R) > 200 * 1024) return set_error(XALM_ERR_UNSUPPORTED, "latent_attend: heads need too much shared memory");
	Pool pool;
	auto put_w = [&](const float* src, size_t cnt) -> void* {
		if (!w_bf16) return pool.put(src, cnt);
		std::vector<uint16_t> wb(cnt);
		for (size_t i = 0; i < cnt; i++) wb[i] = bf16_bits(src[i]);
		return pool.put(wb.data(), cnt);
	};
	std::vector<float> ukT((size_t) H * R * d); // uk (H d, R) as H matrices (R, d)
	for (int h = 0; h < H; h++)
		for (int i = 0; i < d; i++)
			for (int j = 0; j < R; j++) ukT[((size_t) h * R + j) * d + i] = uk[((size_t) h * d + i) * R + j];
	void* d_cache;
	if (cache_bf16) {
		std::vector<uint16_t> cb((size_t) n * ld);
		for (size_t i = 0; i < cb.size(); i++) cb[i] = bf16_bits(cache[i]);
		d_cache = pool.put(cb.data(), cb.size());
	} else d_cache = pool.put(cache, (size_t) n * ld);
	const SeqStep st = {pos0, T};
	const SeqStep* d_st = pool.put(&st, 1);
	const float* d_q = pool.put(q, (size_t) T * H * (d + r));
	const float* d_gate = pool.put(gate, (size_t) T * H * dv);
	const float* d_freq = pool.put(freq, (size_t) r / 2);
	void *d_ukT = put_w(ukT.data(), ukT.size()), *d_uv = put_w(uv, (size_t) H * dv * R);
	float *qabs = pool.raw<float>((size_t) T * H * da), *olat = pool.raw<float>((size_t) T * H * R), *d_out = pool.raw<float>((size_t) T * H * dv);
	if (!d_cache || !d_st || !d_q || !d_ukT || !d_uv || !qabs || !olat || !d_out || (gate && !d_gate) || (r && !d_freq))
		return set_error(XALM_ERR_CUDA, "latent_attend: device allocation failed");
	RowsEpi eb;
	eb.kind = EPI_STORE; eb.out = qabs; eb.ldo = H * da; eb.batch_a = d + r; eb.batch_w = (size_t) R * d; eb.batch_o = da;
	XALM_TRY(launch_rows(d_q, H * (d + r), d_ukT, w_bf16 != 0, T, R, d, eb, nullptr, H));
	if (r) {
		RopeHeadsArgs ra = {};
		ra.src = d_q; ra.lds = H * (d + r); ra.src_off = d; ra.src_stride = d + r;
		ra.dst = qabs; ra.ldd = H * da; ra.dst_off = R; ra.dst_stride = da;
		ra.heads = H; ra.n = r; ra.rot_half = r / 2; ra.freq = d_freq; ra.step = d_st;
		XALM_TRY(launch_rope_heads(ra, T, nullptr));
	}
	SwaArgs sa = {};
	sa.q = qabs; sa.ldq = H * da;
	sa.kc = d_cache; sa.vc = d_cache; sa.ldk = ld; sa.ldv = ld; sa.ring = n;
	sa.H = H; sa.G = 1; sa.d = da; sa.dv = R; sa.window = 0x7fffffff; sa.scale = scale;
	sa.step = d_st; sa.out = olat;
	sa.n_splits = n_splits;
	const int cap = std::max(4 * 64, 4 * T);
	sa.part_cap = n_splits ? T * n_splits : cap;
	sa.part_o = pool.raw<float>((size_t) sa.part_cap * H * R);
	sa.part_ml = pool.raw<float>((size_t) sa.part_cap * H * 2);
	sa.tickets = pool.raw<unsigned>((size_t) 8 * T);
	if (!sa.part_o || !sa.part_ml || !sa.tickets) return set_error(XALM_ERR_CUDA, "latent_attend: device allocation failed");
	XALM_TRY(launch_swa(sa, T, cache_bf16 == 0, nullptr));
	RowsEpi ev;
	ev.kind = EPI_STORE; ev.out = d_out; ev.ldo = H * dv; ev.batch_a = R; ev.batch_w = (size_t) dv * R; ev.batch_o = dv;
	if (gate) { ev.mul = d_gate; ev.ldm = H * dv; ev.mul_act = ACT_SIGMOID; }
	XALM_TRY(launch_rows(olat, H * R, d_uv, w_bf16 != 0, T, dv, R, ev, nullptr, H));
	XALM_TRY(finish("latent_attend"));
	XALM_CUDA_CHECK(cudaMemcpy(out, d_out, (size_t) T * H * dv * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}

int xalm_cuda_rows_act(float* out, const float* x, const float* w, int T, int N, int K, int act, float cap, const float* mul, int mul_act, int w_bf16) {
	if (!out || !x || !w || T <= 0 || N <= 0 || K <= 0) return set_error(XALM_ERR_INVALID, "rows_act: bad argument");
	Pool pool;
	void* d_w;
	if (w_bf16) {
		std::vector<uint16_t> wb((size_t) N * K);
		for (size_t i = 0; i < wb.size(); i++) wb[i] = bf16_bits(w[i]);
		d_w = pool.put(wb.data(), wb.size());
	} else d_w = pool.put(w, (size_t) N * K);
	const float* d_x = pool.put(x, (size_t) T * K);
	const float* d_mul = pool.put(mul, (size_t) T * N);
	float* d_out = pool.raw<float>((size_t) T * N);
	if (!d_w || !d_x || !d_out || (mul && !d_mul)) return set_error(XALM_ERR_CUDA, "rows_act: device allocation failed");
	RowsEpi e;
	e.out = d_out; e.ldo = N;
	if (act != ACT_NONE) { e.kind = EPI_ACT; e.act = act; }
	else { e.kind = EPI_STORE; e.cap = cap; e.mul = d_mul; e.ldm = N; e.mul_act = mul_act; }
	XALM_TRY(launch_rows(d_x, K, d_w, w_bf16 != 0, T, N, K, e, nullptr));
	XALM_TRY(finish("rows_act"));
	XALM_CUDA_CHECK(cudaMemcpy(out, d_out, (size_t) T * N * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}


int xalm_cuda_sink_attention(float* out, const float* q, const float* k, const float* v, int T, int pos0, int H, int G, int d, int dv, float scale,
                             const float* sink, float out_scale, int n_splits, int cache_bf16) {
	return swa_attention_op(out, q, nullptr, k, v, T, pos0, H, G, d, dv, 0x7fffffff, 0, scale, 0.f, nullptr, nullptr, nullptr, pos0 + T, n_splits, cache_bf16, sink,
	                        out_scale);
}

int xalm_cuda_norm_conv(float* out, float* hist, const float* x, int T, int W, int groups, int taps, int readers, const float* w, const float* cw, float eps) {
	if (!out || !hist || !x || !w || !cw || T <= 0 || W <= 0 || readers < 1 || readers > 2) return set_error(XALM_ERR_INVALID, "norm_conv: bad argument");
	Pool pool;
	const size_t hw = (size_t) std::max(taps - 1, 1) * W;
	const SeqStep st = {0, T};
	NormConvArgs a = {};
	a.x = pool.put(x, (size_t) T * W); a.width = W; a.groups = groups; a.taps = taps; a.readers = readers; a.eps = eps;
	const float *d_w = pool.put(w, (size_t) readers * W), *d_cw = pool.put(cw, (size_t) readers * W * taps);
	float *d_hist = pool.put(hist, readers * hw), *d_stage = pool.raw<float>(readers * hw), *d_out = pool.raw<float>((size_t) readers * T * W);
	a.step = pool.put(&st, 1);
	if (!a.x || !d_w || !d_cw || !d_hist || !d_stage || !d_out || !a.step) return set_error(XALM_ERR_CUDA, "norm_conv: device allocation failed");
	for (int r = 0; r < readers; r++) {
		a.w[r] = d_w + (size_t) r * W; a.cw[r] = d_cw + (size_t) r * W * taps;
		a.hist[r] = d_hist + r * hw; a.stage[r] = d_stage + r * hw; a.out[r] = d_out + (size_t) r * T * W;
	}
	XALM_TRY(norm_conv_prepare(W, taps, groups));
	XALM_TRY(launch_norm_conv(a, T, nullptr));
	XALM_TRY(finish("norm_conv"));
	XALM_CUDA_CHECK(cudaMemcpy(out, d_out, (size_t) readers * T * W * 4, cudaMemcpyDeviceToHost));
	XALM_CUDA_CHECK(cudaMemcpy(hist, d_hist, readers * hw * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}

int xalm_cuda_short_conv(float* out, float* hist, const float* x, int T, int C, int taps, const float* w, const float* bias, int act) {
	if (!out || !hist || !x || !w || T <= 0 || C <= 0) return set_error(XALM_ERR_INVALID, "short_conv: bad argument");
	Pool pool;
	const size_t hw = (size_t) std::max(taps - 1, 1) * C;
	const SeqStep st = {0, T};
	ShortConvArgs a = {};
	a.in = pool.put(x, (size_t) T * C); a.ld_in = C; a.ld_out = C; a.C = C; a.taps = taps;
	a.out = pool.raw<float>((size_t) T * C);
	a.w = pool.put(w, (size_t) C * taps); a.bias = pool.put(bias, (size_t) C); a.act = act;
	a.hist = pool.put(hist, hw); a.stage = pool.raw<float>(hw);
	a.step = pool.put(&st, 1);
	if (!a.in || !a.out || !a.w || !a.hist || !a.stage || !a.step) return set_error(XALM_ERR_CUDA, "short_conv: device allocation failed");
	XALM_TRY(launch_short_conv(a, T, nullptr));
	XALM_TRY(finish("short_conv"));
	XALM_CUDA_CHECK(cudaMemcpy(out, a.out, (size_t) T * C * 4, cudaMemcpyDeviceToHost));
	XALM_CUDA_CHECK(cudaMemcpy(hist, a.hist, hw * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}

int xalm_cuda_embed_pair(float* out, const int* tokens, int T, int prev, const float* table, int vocab, const float* pair, int buckets, int mul_prev,
                         int mul_cur, float scale, const float* w, int groups, int W, float eps) {
	if (!out || !tokens || !table || T <= 0 || vocab <= 0 || W <= 0) return set_error(XALM_ERR_INVALID, "embed_pair: bad argument");
	Pool pool;
	const SeqStep st = {0, T, prev};
	EmbedPairArgs a = {};
	a.table = pool.put(table, (size_t) vocab * W); a.pair = pool.put(pair, (size_t) (buckets + 1) * W);
	a.scale = scale; a.mul_prev = mul_prev; a.mul_cur = mul_cur; a.buckets = buckets;
	a.w = pool.put(w, (size_t) W); a.groups = groups; a.width = W; a.eps = eps;
	a.tokens = pool.put(tokens, (size_t) T); a.step = pool.put(&st, 1);
	a.x = pool.raw<float>((size_t) T * W);
	if (!a.table || !a.tokens || !a.step || !a.x || (pair && !a.pair)) return set_error(XALM_ERR_CUDA, "embed_pair: device allocation failed");
	XALM_TRY(launch_embed_pair(a, false, T, nullptr));
	XALM_TRY(finish("embed_pair"));
	XALM_CUDA_CHECK(cudaMemcpy(out, a.x, (size_t) T * W * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}

int xalm_cuda_keyed_recurrence(float* out, float* state, const float* q, const float* k, const float* v, const float* f, int T, int H, int rep, int d, int dv,
                               int mode, float q_scale, const float* dt_bias, const float* A_log, const float* skip, const float* norm_w, const float* gate,
                               float eps) {
	if (!out || !state || !q || !k || !v || !f || T <= 0 || H <= 0 || rep <= 0 || H % rep || d <= 0 || dv <= 0 || (mode != 1 && mode != 2) ||
	    (mode == 2 && (!dt_bias || !A_log)))
		return set_error(XALM_ERR_INVALID, "keyed_recurrence: bad argument");
	const size_t smem = hgrn2_smem_bytes(d, dv);
	if (!hgrn2_cols_ok(d, dv, T, true) && (smem > 200 * 1024 || dv > 1024)) return set_error(XALM_ERR_UNSUPPORTED, "keyed_recurrence: a head's state needs %zu bytes of shared memory", smem);
	Pool pool;
	const int nqk = H / rep * d, nf = mode == 1 ? H * d : H;
	const int ld = 2 * nqk + 2 * H * dv + nf; // q | k | v | gate | decays or step sizes
	std::vector<float> proj((size_t) T * ld, 0.f);
	for (int t = 0; t < T; t++) {
		float* row = &proj[(size_t) t * ld];
		memcpy(row, q + (size_t) t * nqk, (size_t) nqk * 4);
		memcpy(row + nqk, k + (size_t) t * nqk, (size_t) nqk * 4);
		memcpy(row + 2 * nqk, v + (size_t) t * H * dv, (size_t) H * dv * 4);
		if (gate) memcpy(row + 2 * nqk + H * dv, gate + (size_t) t * H * dv, (size_t) H * dv * 4);
		memcpy(row + 2 * nqk + 2 * H * dv, f + (size_t) t * nf, (size_t) nf * 4);
	}
	const SeqStep st = {0, T};
	Hgrn2Args a = {};
	a.proj = pool.put(proj.data(), proj.size()); a.ld = ld; a.q_off = 0; a.k_off = nqk; a.v_off = 2 * nqk;
	a.f_off = a.dt_off = 2 * nqk + 2 * H * dv;
	a.H = H; a.d = d; a.dv = dv; a.keyed = mode; a.qk_rep = rep; a.q_scale = q_scale;
	a.dt_bias = pool.put(dt_bias, (size_t) H); a.A_log = pool.put(A_log, (size_t) H); a.skip = pool.put(skip, (size_t) H);
	a.norm_w = pool.put(norm_w, (size_t) dv); a.eps = eps;
	if (gate) { a.gate = a.proj; a.ldg = ld; a.g_off = 2 * nqk + H * dv; }
	a.state = pool.put(state, (size_t) H * d * dv);
	a.step = pool.put(&st, 1);
	a.out = pool.raw<float>((size_t) T * H * dv);
	a.max_rows = T;
	if (!a.proj || !a.state || !a.step || !a.out) return set_error(XALM_ERR_CUDA, "keyed_recurrence: device allocation failed");
	XALM_TRY(hgrn2_prepare(d, dv));
	XALM_TRY(launch_hgrn2(a, nullptr));
	XALM_TRY(finish("keyed_recurrence"));
	XALM_CUDA_CHECK(cudaMemcpy(out, a.out, (size_t) T * H * dv * 4, cudaMemcpyDeviceToHost));
	XALM_CUDA_CHECK(cudaMemcpy(state, a.state, (size_t) H * d * dv * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}

int xalm_cuda_rows_act_bias(float* out, const float* x, const float* w, int T, int N, int K, int act, const float* bias, float act_pow, int w_bf16) {
	if (!out || !x || !w || T <= 0 || N <= 0 || K <= 0) return set_error(XALM_ERR_INVALID, "rows_act_bias: bad argument");
	Pool pool;
	void* d_w;
	if (w_bf16) {
		std::vector<uint16_t> wb((size_t) N * K);
		for (size_t i = 0; i < wb.size(); i++) wb[i] = bf16_bits(w[i]);
		d_w = pool.put(wb.data(), wb.size());
	} else d_w = pool.put(w, (size_t) N * K);
	const float* d_x = pool.put(x, (size_t) T * K);
	float* d_out = pool.raw<float>((size_t) T * N);
	RowsEpi e;
	e.kind = EPI_ACT; e.act = act; e.bias = pool.put(bias, (size_t) N); e.act_pow = act_pow; e.out = d_out; e.ldo = N;
	if (!d_w || !d_x || !d_out || (bias && !e.bias)) return set_error(XALM_ERR_CUDA, "rows_act_bias: device allocation failed");
	XALM_TRY(launch_rows(d_x, K, d_w, w_bf16 != 0, T, N, K, e, nullptr));
	XALM_TRY(finish("rows_act_bias"));
	XALM_CUDA_CHECK(cudaMemcpy(out, d_out, (size_t) T * N * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}

int xalm_cuda_gated_group_norm(float* out, const float* y, const float* gate, const float* w, int T, int W, int groups, float eps, float out_scale, int ld_out) {
	if (!out || !y || !w || T <= 0 || W <= 0 || ld_out < W) return set_error(XALM_ERR_INVALID, "gated_group_norm: bad argument");
	Pool pool;
	GroupNormArgs g;
	g.y = pool.put(y, (size_t) T * W); g.ldy = W;
	g.gate = pool.put(gate, (size_t) T * W); g.ldg = W;
	g.w = pool.put(w, (size_t) W); g.groups = groups; g.width = W; g.eps = eps; g.out_scale = out_scale;
	g.x_out = pool.raw<float>((size_t) T * ld_out); g.ld_out = ld_out;
	if (!g.y || !g.w || !g.x_out || (gate && !g.gate)) return set_error(XALM_ERR_CUDA, "gated_group_norm: device allocation failed");
	XALM_TRY(group_norm_prepare(W, groups));
	XALM_TRY(launch_group_norm(g, T, nullptr));
	XALM_TRY(finish("gated_group_norm"));
	XALM_CUDA_CHECK(cudaMemcpy(out, g.x_out, (size_t) T * ld_out * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}

} // extern "C"
