// kubolorn.cu — the Kubolorn family of the model registry (family.h): a decoder described by a config.json whose layers run a token
// mixer and a feed-forward SIDE BY SIDE on the same residual row, x <- x + (mixer(r1(x)) + ff(r2(x))), where a reader r is the grouped RMS
// norm followed by h + conv(h), a depthwise causal convolution over time on the normed rows.  A run of layers may repeat ("loop": the
// same weights, a cache and state of its own per repetition).
//
//   embedding          scaled table row + a hashed row for the (previous token, token) pair, then the grouped norm
//   mixer "gla"        gated linear attention: S_t = diag(alpha_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t d^-1/2 per head, with a decay per key
//                      channel alpha = sigmoid(W_a2 W_a1 h + b)^(1/tau); per-head RMS norm of o with a shared weight, silu gate, W_o
//   mixer "parallel"   two mixers on the same input, summed with fixed scales:
//                      left   softmax attention over grouped key heads whose VALUES ARE THE UNROTATED KEYS; rotary positions on part of each
//                             head with YaRN-rescaled frequencies and magnitude; a learned sink per head in the softmax's denominator
//                      right  state-space duality (Mamba-2): [z | x | B | C | dt] = W_in h; x, B, C through a short convolution and silu;
//                             S_t = exp(-exp(A_log) dt) S_{t-1} + dt B_t x_t^T, y_t = S_t^T C_t + D x_t; y silu(z), grouped norm, W_o
//   feed-forward       dense W_down gelu_tanh(W_up h), or `top` of `experts` small W_down relu(W_up h)^2 weighted by the softmax over the
//                      chosen router logits
//   output             grouped norm, logits = embedding table . row
//
// The step function, graph replay of one-token steps, uploads, release and the C entry points are the shared sequence engine's
// (seq_family.cuh).  Per pass and layer run here:
//     both readers:     norm_conv (one launch: norm, convolution and the carried rows of both)
//     gla:              rows product [q | k | v | g | a1] -> rows product [a2] with the decay's bias, log-sigmoid and power fused -> the
//                       recurrence kernels of mix_ops.cuh in their keyed mode (head norm and gate fused) -> rows product [o] + residual
//     parallel:         rows product [q | k | z | xBC | dt] -> qkv_post (rotation with magnitude, cache rows: rotated keys, unrotated keys as
//                       values) -> swa_attn / swa_tile with the sink -> short_conv (+ silu) -> recurrence kernels, step-size mode (softplus,
//                       decay and skip fused) -> group norm with the gate in front -> ONE rows product [o_left | o_right] on the two results
//                       side by side (their scales applied where they are written) + residual
//     dense ff:         rows product [up, gelu fused] -> rows product [down] + residual
//     experts:          moe_router -> moe_sort -> moe_gemm [up, relu^2 fused] -> moe_gemm [down] -> moe_combine (+ residual)
// The recurrences (with the state-space mixer's convolution and norm) run on the engine's side stream, beside the attention and the
// feed-forward on the main one; the output projection waits for both ("seq_overlap", a branch of the captured one-token graph).
//
// Cache / state manager, per layer RUN: the normed rows of the last taps - 1 positions for both readers; gla: the fp32 state (heads x dim x
// vdim); parallel: one cache row of rotated keys and one of unrotated keys per position, the fp32 state (heads x state x vdim) and the
// convolution's last inputs.  release() zeroes states and carried rows; cache rows need no clearing, a sequence only reads positions it wrote.
//
// Precision: the residual stream, norms, convolutions, rotation angles, scores, softmax and sink, router, decays, step sizes, both
// recurrences with their states, gates and every sum are fp32 in both modes.  XALM_PRECISION_BF16 keeps matrices and the key cache in
// bf16 and sends dense products of long passes through the tcgen05 GEMM (fp16 operands, fp32 accumulation); XALM_PRECISION_F32 widens
// both and uses the fp32 FMA kernels only.
#include "seq_family.cuh"

#include "conv_ops.cuh"
#include "moe_ops.cuh"

namespace xalm {
namespace {

using namespace mix;
using namespace seq;

enum { MIX_GLA = 0, MIX_PARALLEL = 1 };
enum { FF_NONE = 0, FF_DENSE = 1, FF_MOE = 2 };

struct Layer { // weights and sizes; what a sequence holds lives in Run
	int mixer = MIX_GLA, ff_kind = FF_NONE;
	// gla
	int H = 0, d = 0, dv = 0;
	float tau = 1.f;
	float *a2_bias = nullptr, *head_norm = nullptr;
	void* w_a2 = nullptr;
	int off_k = 0, off_v = 0, off_g = 0, off_a1 = 0, off_alpha = 0, rank = 0;
	// parallel, left: aH query heads over aG key heads of ad
	int aH = 0, aG = 0, ad = 0, rot_dims = 0;
	float a_scale = 1.f, rot_mag = 1.f, left_scale = 1.f, right_scale = 1.f;
	std::vector<float> freq_host;
	float *freq = nullptr, *sink = nullptr;
	// parallel, right: sH heads of sP value channels, sG groups of sN state channels
	int sH = 0, sP = 0, sN = 0, sG = 0, s_taps = 0, s_norm_groups = 1;
	int off_z = 0, off_xbc = 0, off_dt = 0, off_conv = 0;
	float *conv_w = nullptr, *conv_b = nullptr, *dt_bias = nullptr, *A_log = nullptr, *D = nullptr, *s_norm = nullptr;
	int n_in = 0, k_o = 0; // columns of the stacked input projection; rows the output projection reads
	// feed-forward
	int ff = 0, E = 0, top = 0;
	void *w_in = nullptr, *w_o = nullptr, *w_up = nullptr, *w_down = nullptr, *w_router = nullptr;
	WMat m_in, m_o, m_up, m_down;
	TcWeight t_in, t_o, t_up, t_down;
	std::vector<TcWeight> t_eup, t_edown; // per expert, when the mixture's long passes run on the tensor cores
	float *norm[2] = {nullptr, nullptr}, *canon[2] = {nullptr, nullptr};
	long long bytes = 0, expert_bytes = 0; // what one run of the layer reads of its matrices; of that, one expert's share
	int inner() const { return sH * sP; }
	int conv_channels() const { return sH * sP + 2 * sG * sN; }
};

struct Run { // one execution of a layer within a pass: the sequence's cache and state there
	int layer = 0;
	float* hist = nullptr;      // (2, taps - 1, width) normed rows of the last positions, mixer's reader then feed-forward's
	float* state = nullptr;     // gla (H, d, dv); parallel (sH, sN, sP)
	float* conv_hist = nullptr; // parallel (s_taps - 1, conv channels)
	void *kc = nullptr, *vc = nullptr; // parallel (max_tokens, aG * ad) rotated keys; unrotated keys = values
};

struct KubolornModel : SeqModel {
	float embed_scale = 1.f;
	int groups = 1, taps = 1, buckets = 0;
	long long mul_prev = 0, mul_cur = 0;
	void* pair = nullptr;
	float* embed_norm = nullptr;
	std::vector<Layer> layers;
	std::vector<Run> runs;
	// one pass
	float *x = nullptr, *h1 = nullptr, *h2 = nullptr, *hn = nullptr, *proj = nullptr, *att = nullptr, *yssd = nullptr, *ffh = nullptr;
	float *stage_canon = nullptr, *stage_conv = nullptr;
	int proj_ld = 4;
	float *part_o = nullptr, *part_ml = nullptr;
	unsigned* tickets = nullptr;
	int part_cap = 0;
	int *moe_idx = nullptr, *moe_sorted = nullptr, *moe_tiles = nullptr, *moe_ntiles = nullptr;
	float *moe_wgt = nullptr, *moe_hid = nullptr, *moe_out = nullptr;
	int *moe_off = nullptr, *moe_inv = nullptr, *h_off = nullptr;
	float* moe_x = nullptr;
};
typedef KubolornModel Kb;

// Rotary frequencies f_i = base^(-2i/dims) with YaRN rescaling: with dim(t) = dims ln(original / (2 pi t)) / (2 ln base) the pairs from
// lo = floor(dim(fast)) to hi = ceil(dim(slow)) are blended, ramp_i = clamp((i - lo) / (hi - lo), 0, 1), f_i <- f_i / factor * ramp_i +
// f_i (1 - ramp_i); cos and sin are then multiplied by 0.1 ln(factor) + 1 (*mag).
std::vector<float> yarn_frequencies(const xjson::Value& rot, int dims, float* mag) {
	const double base = getf(rot, "base");
	const xjson::Value* sc = rot.find("scaling");
	const bool scaled = sc && sc->kind == xjson::Value::Obj;
	double factor = 1, fast = 1, slow = 1, original = 1, lo = 0, hi = 0;
	*mag = 1.f;
	if (scaled) {
		factor = getf(*sc, "factor"); fast = getf(*sc, "fast"); slow = getf(*sc, "slow"); original = getf(*sc, "original");
		auto dim_of = [&](double turns) { return dims * log(original / (2.0 * M_PI * turns)) / (2.0 * log(base)); };
		lo = std::max(floor(dim_of(fast)), 0.0);
		hi = std::min(ceil(dim_of(slow)), (double) dims - 1);
		*mag = (float) (0.1 * log(factor) + 1.0);
	}
	std::vector<float> f((size_t) dims / 2);
	for (int i = 0; i < dims / 2; i++) {
		double fi = pow(base, -2.0 * i / dims);
		if (scaled) {
			const double ramp = std::min(1.0, std::max(0.0, (i - lo) / std::max(hi - lo, 0.001)));
			fi = fi / factor * ramp + fi * (1.0 - ramp);
		}
		f[(size_t) i] = (float) fi;
	}
	return f;
}

// ---- config.json ------------------------------------------------------------------------------------------------------------------
int parse_config(SeqModel* sm, const char* json) {
	Kb* m = static_cast<Kb*>(sm);
	try {
		const xjson::Value c = xjson::Parser::parse(json, strlen(json));
		m->vocab = geti(c, "vocab");
		m->width = geti(c, "width");
		if (m->vocab <= 0 || m->width <= 0) return set_error(XALM_ERR_INVALID, "config: vocab / width must be positive");
		const int W = m->width;
		if (const xjson::Value* nv = c.find("norm"); nv && nv->kind == xjson::Value::Obj) {
			if (nv->contains("eps")) m->eps = (float) getf(*nv, "eps");
			if (nv->contains("groups")) m->groups = geti(*nv, "groups");
		}
		if (m->groups <= 0 || W % m->groups) return set_error(XALM_ERR_INVALID, "config: %d norm groups do not divide a width of %d", m->groups, W);
		if (const xjson::Value* cv = c.find("canon"); cv && cv->kind == xjson::Value::Obj) m->taps = geti(*cv, "taps");
		if (m->taps < 1 || m->taps > CONV_MAX_TAPS + 1) return set_error(XALM_ERR_UNSUPPORTED, "config: canon.taps %d (1 to %d)", m->taps, CONV_MAX_TAPS + 1);
		expect(m, "embed", {m->vocab, W}, true);
		if (const xjson::Value* ev = c.find("embedding"); ev && ev->kind == xjson::Value::Obj) {
			if (ev->contains("scale")) m->embed_scale = (float) getf(*ev, "scale");
			if (const xjson::Value* bg = ev->find("bigram"); bg && bg->kind == xjson::Value::Obj) {
				m->buckets = geti(*bg, "buckets");
				m->mul_prev = (long long) getf(*bg, "mul_prev");
				m->mul_cur = (long long) getf(*bg, "mul_cur");
				if (m->buckets <= 0 || m->mul_prev < 0 || m->mul_cur < 0) return set_error(XALM_ERR_INVALID, "config: embedding.bigram");
				expect(m, "bigram", {m->buckets + 1, W}, true);
			}
		}
		expect(m, "embed.norm", {W}, false);
		const xjson::Value& layers = c.at("layers");
		if (layers.kind != xjson::Value::Array || layers.arr.empty()) return set_error(XALM_ERR_INVALID, "config: no layers");
		for (size_t li = 0; li < layers.arr.size(); li++) {
			const xjson::Value& lv = layers.arr[li];
			const std::string type = lv.at("type").str;
			const xjson::Value& mx = lv.at("mixer");
			const std::string p = "l" + std::to_string(li) + ".";
			Layer L;
			const xjson::Value* mlp = lv.find("mlp");
			if (mlp && mlp->kind != xjson::Value::Obj) mlp = nullptr;
			expect(m, p + "norm1", {W}, false);
			if (mlp) expect(m, p + "norm2", {W}, false);
			if (type == "gla") {
				L.mixer = MIX_GLA;
				L.H = geti(mx, "heads"); L.d = geti(mx, "dim"); L.dv = mx.contains("vdim") ? geti(mx, "vdim") : L.d;
				L.tau = mx.contains("tau") ? (float) getf(mx, "tau") : 1.f;
				if (L.H <= 0 || L.d <= 0 || L.dv <= 0 || !(L.tau > 0.f)) return set_error(XALM_ERR_INVALID, "config: layer %zu: bad mixer sizes", li);
				expect(m, p + "mix.q", {L.H * L.d, W}, true);
				expect(m, p + "mix.k", {L.H * L.d, W}, true);
				expect(m, p + "mix.v", {L.H * L.dv, W}, true);
				expect(m, p + "mix.g", {L.H * L.dv, W}, true);
				expect(m, p + "mix.o", {W, L.H * L.dv}, true);
				expect(m, p + "mix.norm", {L.dv}, false);
				expect(m, p + "mix.a1", {-1, W}, true);          // the decay's inner size is the tensor's
				expect(m, p + "mix.a2", {L.H * L.d, -1}, true);
				expect(m, p + "mix.a2.b", {L.H * L.d}, false);
			} else if (type == "parallel") {
				L.mixer = MIX_PARALLEL;
				const xjson::Value &lf = mx.at("left"), &rg = mx.at("right");
				L.left_scale = mx.contains("left_scale") ? (float) getf(mx, "left_scale") : 1.f;
				L.right_scale = mx.contains("right_scale") ? (float) getf(mx, "right_scale") : 1.f;
				L.aH = geti(lf, "heads"); L.aG = lf.contains("kv_heads") ? geti(lf, "kv_heads") : L.aH; L.ad = geti(lf, "dim");
				if (L.aH <= 0 || L.aG <= 0 || L.aH % L.aG || L.ad <= 0) return set_error(XALM_ERR_INVALID, "config: layer %zu: %d query heads over %d key heads of %d", li, L.aH, L.aG, L.ad);
				if (lf.contains("vdim") && geti(lf, "vdim") != L.ad) return set_error(XALM_ERR_INVALID, "config: layer %zu: values are the keys, vdim %d differs from dim %d", li, geti(lf, "vdim"), L.ad);
				L.a_scale = lf.contains("scale") ? (float) getf(lf, "scale") : 1.f / sqrtf((float) L.ad);
				if (const xjson::Value* rt = lf.find("rot"); rt && rt->kind == xjson::Value::Obj) {
					L.rot_dims = geti(*rt, "dims");
					if (L.rot_dims < 0 || L.rot_dims > L.ad || L.rot_dims % 2) return set_error(XALM_ERR_INVALID, "config: layer %zu: %d rotary dimensions in a head of %d", li, L.rot_dims, L.ad);
					if (L.rot_dims) L.freq_host = yarn_frequencies(*rt, L.rot_dims, &L.rot_mag);
				}
				L.sH = geti(rg, "heads"); L.sP = geti(rg, "vdim"); L.sN = geti(rg, "state"); L.sG = rg.contains("groups") ? geti(rg, "groups") : 1;
				L.s_taps = geti(rg, "conv"); L.s_norm_groups = rg.contains("norm_groups") ? geti(rg, "norm_groups") : 1;
				if (L.sH <= 0 || L.sP <= 0 || L.sN <= 0 || L.sG <= 0 || L.sH % L.sG) return set_error(XALM_ERR_INVALID, "config: layer %zu: %d state-space heads in %d groups", li, L.sH, L.sG);
				if (L.s_taps < 1 || L.s_taps > CONV_MAX_TAPS) return set_error(XALM_ERR_UNSUPPORTED, "config: layer %zu: a convolution of %d taps (1 to %d)", li, L.s_taps, CONV_MAX_TAPS);
				if (L.s_norm_groups <= 0 || L.inner() % L.s_norm_groups) return set_error(XALM_ERR_INVALID, "config: layer %zu: %d norm groups do not divide %d", li, L.s_norm_groups, L.inner());
				expect(m, p + "mix.left.q", {L.aH * L.ad, W}, true);
				expect(m, p + "mix.left.k", {L.aG * L.ad, W}, true);
				expect(m, p + "mix.left.sink", {L.aH}, false);
				expect(m, p + "mix.left.o", {W, L.aH * L.ad}, true);
				expect(m, p + "mix.right.in", {2 * L.inner() + 2 * L.sG * L.sN + L.sH, W}, true);
				expect(m, p + "mix.right.conv", {L.conv_channels(), L.s_taps}, false);
				expect(m, p + "mix.right.conv.b", {L.conv_channels()}, false);
				expect(m, p + "mix.right.dt_bias", {L.sH}, false);
				expect(m, p + "mix.right.A_log", {L.sH}, false);
				expect(m, p + "mix.right.D", {L.sH}, false);
				expect(m, p + "mix.right.norm", {L.inner()}, false);
				expect(m, p + "mix.right.o", {W, L.inner()}, true);
			} else return set_error(XALM_ERR_UNSUPPORTED, "config: layer %zu has mixer type '%s' (this family runs 'gla' and 'parallel')", li, type.c_str());
			if (mlp) {
				const std::string kind = mlp->contains("kind") ? mlp->at("kind").str : "dense";
				if (kind == "dense") {
					L.ff_kind = FF_DENSE;
					L.ff = geti(*mlp, "ff");
					if (L.ff <= 0) return set_error(XALM_ERR_INVALID, "config: layer %zu: ff", li);
					expect(m, p + "mlp.up", {L.ff, W}, true);
					expect(m, p + "mlp.down", {W, L.ff}, true);
				} else if (kind == "moe") {
					L.ff_kind = FF_MOE;
					L.ff = geti(mlp->at("expert"), "ff");
					const xjson::Value& r = mlp->at("router");
					L.E = geti(r, "experts");
					L.top = geti(r, "top");
					if (L.ff <= 0 || L.E <= 0 || L.top <= 0 || L.top > L.E) return set_error(XALM_ERR_INVALID, "config: layer %zu: %d of %d experts of %d", li, L.top, L.E, L.ff);
					for (int e = 0; e < L.E; e++) {
						const std::string pe = p + "mlp.e" + std::to_string(e) + ".";
						expect(m, pe + "up", {L.ff, W}, true);
						expect(m, pe + "down", {W, L.ff}, true);
					}
					expect(m, p + "mlp.router", {L.E, W}, true);
				} else return set_error(XALM_ERR_UNSUPPORTED, "config: layer %zu has feed-forward kind '%s'", li, kind.c_str());
			}
			expect(m, p + "canon1", {W, m->taps}, false);
			if (mlp) expect(m, p + "canon2", {W, m->taps}, false);
			m->layers.push_back(std::move(L));
		}
		// the order the layers run in: layers start .. stop - 1 `times` times in a row, then the rest
		const int nl = (int) m->layers.size();
		int start = 0, stop = 0, times = 1;
		if (const xjson::Value* lp = c.find("loop"); lp && lp->kind == xjson::Value::Obj) {
			start = geti(*lp, "start"); stop = geti(*lp, "stop"); times = lp->contains("times") ? geti(*lp, "times") : 1;
			if (start < 0 || stop < start || stop > nl || times < 1) return set_error(XALM_ERR_INVALID, "config: loop over layers [%d, %d) %d times", start, stop, times);
		}
		for (int li = 0; li < nl; li++) {
			if (li == start && stop > start)
				for (int r = 0; r < times; r++)
					for (int lj = start; lj < stop; lj++) { Run R; R.layer = lj; m->runs.push_back(R); }
			if (li < start || li >= stop) { Run R; R.layer = li; m->runs.push_back(R); }
		}
		m->n_layers = (int) m->runs.size(); // what read_state counts: layer runs
		expect(m, "final.norm", {W}, false);
	} catch (const std::exception& e) {
		return set_error(XALM_ERR_INVALID, "config.json: %s", e.what());
	}
	return XALM_OK;
}

// ---- the kernels of one pass ----------------------------------------------------------------------------------------------------------
RowsEpi residual_epi(Kb* m) { // x <- x + product
	RowsEpi e;
	e.kind = EPI_HC;
	e.xs = m->x;
	e.S = 1;
	e.stream_stride = (size_t) m->chunk * m->width;
	return e;
}

// What of a layer does not depend on the rest runs on the side stream (a branch of the one-token graph): the recurrences, which keep few SMs
// busy for long, beside the attention and the feed-forward's products.  The side stream never runs a matrix product: the tensor-core path's
// operand planes belong to the main stream.
struct Fork {
	Kb* m;
	bool on;
	cudaStream_t side() const { return on ? m->side : m->stream; }
	int open() const {
		if (!on) return XALM_OK;
		XALM_CUDA_CHECK(cudaEventRecord(m->ev_fork, m->stream));
		XALM_CUDA_CHECK(cudaStreamWaitEvent(m->side, m->ev_fork, 0));
		return XALM_OK;
	}
	int mark() const { // the side branch ends here
		if (on) XALM_CUDA_CHECK(cudaEventRecord(m->ev_join, m->side));
		return XALM_OK;
	}
	int join() const {
		if (on) XALM_CUDA_CHECK(cudaStreamWaitEvent(m->stream, m->ev_join, 0));
		return XALM_OK;
	}
};

// input projections on the main stream, then the recurrence on the fork's side
int enqueue_gla(Kb* m, const Layer& L, const Run& R, int n, const Fork& fk, int* nl) {
	const int H = L.H, d = L.d, dv = L.dv;
	RowsEpi est;
	est.kind = EPI_STORE; est.out = m->proj; est.ldo = m->proj_ld;
	XALM_TRY(rows_product(m, m->h1, m->width, L.w_in, &L.t_in, n, L.n_in, m->width, est, nl));
	RowsEpi ea; // alpha = sigmoid(W_a2 (W_a1 h) + b)^(1 / tau)
	ea.kind = EPI_ACT; ea.act = ACT_SIGMOID_POW; ea.act_pow = 1.f / L.tau; ea.bias = L.a2_bias; ea.out = m->proj + L.off_alpha; ea.ldo = m->proj_ld;
	XALM_TRY(rows_product(m, m->proj + L.off_a1, m->proj_ld, L.w_a2, nullptr, n, H * d, L.rank, ea, nl));
	Hgrn2Args ha = {};
	ha.proj = m->proj; ha.ld = m->proj_ld; ha.q_off = 0; ha.k_off = L.off_k; ha.v_off = L.off_v; ha.f_off = L.off_alpha;
	ha.H = H; ha.d = d; ha.dv = dv;
	ha.keyed = 1; ha.qk_rep = 1; ha.q_scale = 1.f / sqrtf((float) d);
	ha.norm_w = L.head_norm; ha.eps = m->eps;
	ha.gate = m->proj; ha.ldg = m->proj_ld; ha.g_off = L.off_g;
	ha.state = R.state; ha.step = m->d_step; ha.out = m->att; ha.max_rows = m->chunk;
	XALM_TRY(fk.open());
	XALM_TRY(launch_hgrn2(ha, fk.side()));
	(*nl)++;
	return fk.mark();
}

// input projection on the main stream; the state-space mixer on the fork's side; the attention on the main stream
int enqueue_parallel(Kb* m, const Layer& L, const Run& R, int n, const Fork& fk, int* nl) {
	cudaStream_t s = m->stream;
	const bool f32 = m->precision == XALM_PRECISION_F32;
	const int H = L.aH, G = L.aG, d = L.ad;
	RowsEpi est;
	est.kind = EPI_STORE; est.out = m->proj; est.ldo = m->proj_ld;
	XALM_TRY(rows_product(m, m->h1, m->width, L.w_in, &L.t_in, n, L.n_in, m->width, est, nl));
	// right: convolution + silu on x | B | C, the recurrence, gate and grouped norm into the columns behind the attention's result
	XALM_TRY(fk.open());
	cudaStream_t side = fk.side();
	int launches = 1;
	ShortConvArgs ca = {};
	ca.in = m->proj; ca.ld_in = m->proj_ld; ca.in_off = L.off_xbc;
	ca.out = m->proj; ca.ld_out = m->proj_ld; ca.out_off = L.off_conv;
	ca.C = L.conv_channels(); ca.taps = L.s_taps; ca.w = L.conv_w; ca.bias = L.conv_b; ca.act = ACT_SILU;
	ca.hist = R.conv_hist; ca.stage = m->stage_conv; ca.step = m->d_step;
	XALM_TRY(launch_short_conv(ca, n, side, &launches));
	*nl += launches;
	Hgrn2Args ha = {};
	ha.proj = m->proj; ha.ld = m->proj_ld;
	ha.v_off = L.off_conv; ha.k_off = L.off_conv + L.inner(); ha.q_off = ha.k_off + L.sG * L.sN;
	ha.H = L.sH; ha.d = L.sN; ha.dv = L.sP;
	ha.keyed = 2; ha.qk_rep = L.sH / L.sG; ha.dt_off = L.off_dt; ha.dt_bias = L.dt_bias; ha.A_log = L.A_log; ha.skip = L.D;
	ha.eps = m->eps;
	ha.state = R.state; ha.step = m->d_step; ha.out = m->yssd; ha.max_rows = m->chunk;
	XALM_TRY(launch_hgrn2(ha, side));
	(*nl)++;
	GroupNormArgs g;
	g.y = m->yssd; g.ldy = L.inner();
	g.gate = m->proj + L.off_z; g.ldg = m->proj_ld;
	g.w = L.s_norm; g.groups = L.s_norm_groups; g.width = L.inner(); g.eps = m->eps;
	g.out_scale = L.right_scale;
	g.x_out = m->att + H * d; g.ld_out = L.k_o;
	XALM_TRY(launch_group_norm(g, n, side));
	(*nl)++;
	XALM_TRY(fk.mark());
	// left: rotate q in place, rotated keys and (as values) the keys as projected into the cache rows of the step's positions
	QkvPostArgs qa = {};
	qa.proj = m->proj; qa.ld = m->proj_ld; qa.q_off = 0; qa.k_off = H * d; qa.v_off = H * d;
	qa.H = H; qa.G = G; qa.d = d; qa.dv = d;
	qa.freq = L.freq; qa.rot_half = L.rot_dims / 2; qa.rot_mag = L.rot_mag;
	qa.eps = m->eps;
	qa.kc = R.kc; qa.vc = R.vc; qa.cache_f32 = f32; qa.keep_first = 0; qa.ring = m->max_tokens;
	qa.step = m->d_step;
	XALM_TRY(launch_qkv_post(qa, n, s));
	(*nl)++;
	SwaArgs sa = {};
	sa.q = m->proj; sa.ldq = m->proj_ld; sa.q_off = 0;
	sa.kc = R.kc; sa.vc = R.vc; sa.ring = m->max_tokens; sa.keep_first = 0;
	sa.H = H; sa.G = G; sa.d = d; sa.dv = d;
	sa.window = 0x7fffffff; sa.scale = L.a_scale; sa.sink = L.sink; sa.out_scale = L.left_scale;
	sa.step = m->d_step; sa.out = m->att; sa.ldo = L.k_o;
	sa.n_splits = 0;
	sa.part_o = m->part_o; sa.part_ml = m->part_ml; sa.part_cap = m->part_cap; sa.tickets = m->tickets;
	launches = 1;
	XALM_TRY(launch_swa(sa, n, f32, s, &launches));
	*nl += launches;
	return XALM_OK;
}

int enqueue_experts(Kb* m, const Layer& L, int n, int* nl) {
	cudaStream_t s = m->stream;
	const int W = m->width;
	MoeRouteArgs ra = {};
	ra.h = m->h2; ra.ldh = W; ra.w = L.w_router; ra.w_bf16 = m->w_bf16;
	ra.E = L.E; ra.top = L.top; ra.K = W;
	ra.idx = m->moe_idx; ra.wgt = m->moe_wgt; ra.step = m->d_step;
	// the largest logits are the largest softmax scores; the chosen scores over their sum are the softmax over the chosen logits
	ra.score_kind = MOE_SCORE_SOFTMAX; ra.group_kind = MOE_GROUP_MAX; ra.renormalise = 1; ra.renorm_eps = 0.f;
	XALM_TRY(launch_moe_router(ra, n, s));
	(*nl)++;
	const bool on_tc = m->use_tc && !L.t_eup.empty() && n >= m->tc_min_rows;
	const bool tiled = on_tc || n * L.top > MOE_MATVEC_PAIRS; // steps of a few tokens run one matvec per (token, slot) pair and need no tile list
	if (tiled) {
		MoeSortArgs so = {m->moe_idx, L.top, L.E, m->d_step, m->moe_sorted, m->moe_tiles, m->moe_ntiles, m->moe_off, m->moe_inv};
		XALM_TRY(launch_moe_sort(so, s));
		(*nl)++;
	}
	RowsEpi eu;
	eu.kind = EPI_ACT; eu.act = ACT_RELU_SQUARED; eu.ldo = L.ff;
	if (on_tc) {
		// Long passes of the 16-bit mode: each expert's rows, gathered one after the other, go through the tcgen05 GEMM on that expert's
		// resident fp16 tiles.  How many rows each expert got is read back first (one small copy and a wait per mixture layer and pass).
		XALM_CUDA_CHECK(cudaMemcpyAsync(m->h_off, m->moe_off, (size_t) (L.E + 1) * 4, cudaMemcpyDeviceToHost, s));
		moe_gather_kernel<<<n * L.top, 256, 0, s>>>(m->h2, W, L.top, m->moe_sorted, m->d_step, L.top, W, m->moe_x);
		XALM_SEQ_LAUNCH_CHECK("moe_gather");
		XALM_CUDA_CHECK(cudaStreamSynchronize(s));
		for (int e = 0; e < L.E; e++) {
			const int at = m->h_off[e], cnt = m->h_off[e + 1] - at;
			if (cnt <= 0) continue;
			XALM_TRY(tc_gemm(L.t_eup[(size_t) e], m->moe_x + (size_t) at * W, cnt, m->tc_out, L.ff, m->a_hi, m->a_lo, s));
			eu.out = m->moe_hid + (size_t) at * L.ff;
			XALM_TRY(launch_rows_epilogue(m->tc_out, L.ff, cnt, L.ff, eu, s));
			XALM_TRY(tc_gemm(L.t_edown[(size_t) e], m->moe_hid + (size_t) at * L.ff, cnt, m->moe_out + (size_t) at * W, W, m->a_hi, m->a_lo, s));
			*nl += 5;
		}
	} else {
		MoeGemmArgs ga = {};
		ga.A = m->h2; ga.lda = W; ga.a_div = L.top; ga.W = L.w_up; ga.N = L.ff; ga.K = W;
		ga.sorted = m->moe_sorted; ga.tiles = m->moe_tiles; ga.n_tiles = m->moe_ntiles;
		ga.idx = m->moe_idx; ga.step = m->d_step; ga.top = L.top;
		ga.e = eu; ga.e.out = m->moe_hid;
		XALM_TRY(launch_moe_gemm(ga, m->w_bf16, n * L.top, L.E, s));
		ga.A = m->moe_hid; ga.lda = L.ff; ga.a_div = 1; ga.W = L.w_down; ga.N = W; ga.K = L.ff;
		ga.e = RowsEpi();
		ga.e.kind = EPI_STORE; ga.e.out = m->moe_out; ga.e.ldo = W;
		XALM_TRY(launch_moe_gemm(ga, m->w_bf16, n * L.top, L.E, s));
		*nl += 2;
	}
	MoeCombineArgs ca = {};
	ca.y = m->moe_out; ca.ldy = W; ca.top = L.top; ca.width = W; ca.wgt = m->moe_wgt; ca.part_row = on_tc ? m->moe_inv : nullptr;
	ca.x_in = m->x; ca.x_out = m->x; ca.step = m->d_step;
	XALM_TRY(launch_moe_combine(ca, n, s));
	(*nl)++;
	return XALM_OK;
}

int enqueue_pass(SeqModel* sm, int n, int want, int* nl) {
	Kb* m = static_cast<Kb*>(sm);
	cudaStream_t s = m->stream;
	const int W = m->width;
	const size_t hs = (size_t) m->chunk * W;
	EmbedPairArgs ea = {};
	ea.table = m->embed; ea.pair = m->pair; ea.scale = m->embed_scale; ea.mul_prev = m->mul_prev; ea.mul_cur = m->mul_cur; ea.buckets = m->buckets;
	ea.w = m->embed_norm; ea.groups = m->groups; ea.width = W; ea.eps = m->eps;
	ea.tokens = m->d_tokens; ea.step = m->d_step; ea.x = m->x;
	XALM_TRY(launch_embed_pair(ea, m->w_bf16, n, s));
	(*nl)++;
	for (size_t ri = 0; ri < m->runs.size(); ri++) {
		const Run& R = m->runs[ri];
		const Layer& L = m->layers[(size_t) R.layer];
		const size_t hw = (size_t) (m->taps - 1) * W;
		NormConvArgs na = {};
		na.x = m->x; na.width = W; na.groups = m->groups; na.taps = m->taps; na.readers = L.ff_kind == FF_NONE ? 1 : 2; na.eps = m->eps;
		for (int r = 0; r < 2; r++) {
			na.w[r] = L.norm[r]; na.cw[r] = L.canon[r];
			na.hist[r] = R.hist + r * hw; na.stage[r] = m->stage_canon + r * hw;
		}
		na.out[0] = m->h1; na.out[1] = m->h2;
		na.step = m->d_step;
		int launches = 1;
		XALM_TRY(launch_norm_conv(na, n, s, &launches));
		*nl += launches;
		const Fork fk = {m, tune("seq_overlap") != 0};
		if (L.mixer == MIX_GLA) XALM_TRY(enqueue_gla(m, L, R, n, fk, nl));
		else XALM_TRY(enqueue_parallel(m, L, R, n, fk, nl));
		if (L.ff_kind == FF_DENSE) {
			RowsEpi eu;
			eu.kind = EPI_ACT; eu.act = ACT_GELU_TANH; eu.out = m->ffh; eu.ldo = L.ff;
			XALM_TRY(rows_product(m, m->h2, W, L.w_up, &L.t_up, n, L.ff, W, eu, nl));
			XALM_TRY(rows_product(m, m->ffh, L.ff, L.w_down, &L.t_down, n, W, L.ff, residual_epi(m), nl));
		} else if (L.ff_kind == FF_MOE) XALM_TRY(enqueue_experts(m, L, n, nl));
		XALM_TRY(fk.join());
		XALM_TRY(rows_product(m, m->att, L.k_o, L.w_o, &L.t_o, n, W, L.k_o, residual_epi(m), nl));
		if (m->keep_layers) XALM_CUDA_CHECK(cudaMemcpyAsync(m->layer_sums + ri * hs, m->x, (size_t) n * W * 4, cudaMemcpyDeviceToDevice, s));
	}
	if (want) {
		const int rows = want == 2 ? n : 1, first = want == 2 ? 0 : n - 1;
		GroupNormArgs g;
		g.y = m->x + (size_t) first * W; g.ldy = W;
		g.w = m->final_norm; g.groups = m->groups; g.width = W; g.eps = m->eps;
		g.x_out = m->hn;
		XALM_TRY(launch_group_norm(g, rows, s));
		(*nl)++;
		RowsEpi eh;
		eh.kind = EPI_STORE; eh.out = m->logits; eh.ldo = m->vocab;
		XALM_TRY(rows_product(m, m->hn, W, m->w_head, &m->t_head, rows, m->vocab, W, eh, nl));
	}
	return XALM_OK;
}

// ---- device layouts, cache, state, pass buffers ---------------------------------------------------------------------------------------
int finalize(SeqModel* sm) {
	Kb* m = static_cast<Kb*>(sm);
	const int W = m->width;
	const size_t C = (size_t) m->chunk;
	auto T = [&](const std::string& n) { return tensor_or_null(m, n); };
	size_t max_proj = 4, max_att = 1, max_yssd = 1, max_ff = 1, max_hd = 1, max_h = 1, max_pairs = 0, max_moe_hid = 0, max_conv = 1;
	int max_tiles = 1, max_norm_groups = m->groups, max_norm_width = W;
	bool moe_tc = false;
	const size_t kelem = m->precision == XALM_PRECISION_F32 ? 4 : 2;
	if (m->buckets) XALM_TRY(upload_rows(m, {T("bigram")}, W, false, &m->pair, nullptr));
	XALM_TRY(upload_vec(m, "embed.norm", &m->embed_norm));
	XALM_TRY(norm_conv_prepare(W, m->taps, m->groups));
	for (size_t li = 0; li < m->layers.size(); li++) {
		Layer& L = m->layers[li];
		const std::string p = "l" + std::to_string(li) + ".";
		const long long bytes0 = m->weight_bytes;
		XALM_TRY(upload_vec(m, p + "norm1", &L.norm[0]));
		XALM_TRY(upload_vec(m, p + "canon1", &L.canon[0]));
		if (L.ff_kind != FF_NONE) {
			XALM_TRY(upload_vec(m, p + "norm2", &L.norm[1]));
			XALM_TRY(upload_vec(m, p + "canon2", &L.canon[1]));
		}
		if (L.mixer == MIX_GLA) {
			const int H = L.H, d = L.d, dv = L.dv;
			L.rank = T(p + "mix.a1")->shape[0];
			if (T(p + "mix.a2")->shape[1] != L.rank) return set_error(XALM_ERR_INVALID, "layer %zu: the decay's two matrices meet at %d and %d", li, L.rank, T(p + "mix.a2")->shape[1]);
			L.off_k = H * d; L.off_v = 2 * H * d; L.off_g = L.off_v + H * dv; L.off_a1 = L.off_g + H * dv; L.n_in = L.off_a1 + L.rank;
			L.off_alpha = (L.n_in + 3) / 4 * 4;
			L.k_o = H * dv;
			XALM_TRY(upload_rows(m, {T(p + "mix.q"), T(p + "mix.k"), T(p + "mix.v"), T(p + "mix.g"), T(p + "mix.a1")}, W, false, &L.w_in, &L.m_in));
			XALM_TRY(upload_rows(m, {T(p + "mix.a2")}, L.rank, false, &L.w_a2, nullptr));
			XALM_TRY(upload_vec(m, p + "mix.a2.b", &L.a2_bias));
			XALM_TRY(upload_vec(m, p + "mix.norm", &L.head_norm));
			XALM_TRY(upload_rows(m, {T(p + "mix.o")}, L.k_o, false, &L.w_o, &L.m_o));
			if (!hgrn2_cols_ok(d, dv, m->chunk, true) && hgrn2_smem_bytes(d, dv) > 200 * 1024)
				return set_error(XALM_ERR_UNSUPPORTED, "layer %zu: a recurrent state of %d x %d per head", li, d, dv);
			XALM_TRY(hgrn2_prepare(d, dv));
			max_proj = std::max(max_proj, (size_t) L.off_alpha + H * d);
		} else {
			const int H = L.aH, G = L.aG, d = L.ad, inner = L.inner(), Cc = L.conv_channels();
			L.off_z = H * d + G * d; L.off_xbc = L.off_z + inner; L.off_dt = L.off_xbc + Cc; L.n_in = L.off_dt + L.sH;
			L.off_conv = (L.n_in + 3) / 4 * 4;
			L.k_o = H * d + inner;
			XALM_TRY(upload_rows(m, {T(p + "mix.left.q"), T(p + "mix.left.k"), T(p + "mix.right.in")}, W, false, &L.w_in, &L.m_in));
			XALM_TRY(upload_vec(m, p + "mix.left.sink", &L.sink));
			if (!L.freq_host.empty()) XALM_TRY(upload_floats(m, L.freq_host.data(), L.freq_host.size(), &L.freq));
			XALM_TRY(upload_vec(m, p + "mix.right.conv", &L.conv_w));
			XALM_TRY(upload_vec(m, p + "mix.right.conv.b", &L.conv_b));
			XALM_TRY(upload_vec(m, p + "mix.right.dt_bias", &L.dt_bias));
			XALM_TRY(upload_vec(m, p + "mix.right.A_log", &L.A_log));
			XALM_TRY(upload_vec(m, p + "mix.right.D", &L.D));
			XALM_TRY(upload_vec(m, p + "mix.right.norm", &L.s_norm));
			{ // the two output projections side by side: one product on [left result | right result]
				const HostTensor *ol = T(p + "mix.left.o"), *orr = T(p + "mix.right.o");
				HostTensor both;
				both.shape = {W, L.k_o};
				both.v.resize((size_t) W * L.k_o);
				for (int r = 0; r < W; r++) {
					memcpy(&both.v[(size_t) r * L.k_o], &ol->v[(size_t) r * H * d], (size_t) H * d * 4);
					memcpy(&both.v[(size_t) r * L.k_o + H * d], &orr->v[(size_t) r * inner], (size_t) inner * 4);
				}
				XALM_TRY(upload_rows(m, {&both}, L.k_o, false, &L.w_o, &L.m_o));
			}
			if (!swa_pick_tq(H, G, d, d, m->chunk) && swa_smem_bytes(H, d, d) > 200 * 1024)
				return set_error(XALM_ERR_UNSUPPORTED, "layer %zu: attention heads need %zu bytes of shared memory", li, swa_smem_bytes(H, d, d));
			XALM_TRY(swa_prepare(H, d, d));
			if (!hgrn2_cols_ok(L.sN, L.sP, m->chunk, true) && hgrn2_smem_bytes(L.sN, L.sP) > 200 * 1024)
				return set_error(XALM_ERR_UNSUPPORTED, "layer %zu: a recurrent state of %d x %d per head", li, L.sN, L.sP);
			XALM_TRY(hgrn2_prepare(L.sN, L.sP));
			max_proj = std::max(max_proj, (size_t) L.off_conv + Cc);
			max_yssd = std::max(max_yssd, (size_t) inner);
			max_hd = std::max(max_hd, (size_t) H * d);
			max_h = std::max(max_h, (size_t) H);
			max_conv = std::max(max_conv, (size_t) (L.s_taps - 1) * Cc);
			max_norm_groups = std::max(max_norm_groups, L.s_norm_groups);
			max_norm_width = std::max(max_norm_width, inner);
		}
		max_att = std::max(max_att, (size_t) L.k_o);
		if (L.ff_kind == FF_DENSE) {
			XALM_TRY(upload_rows(m, {T(p + "mlp.up")}, W, false, &L.w_up, &L.m_up));
			XALM_TRY(upload_rows(m, {T(p + "mlp.down")}, L.ff, false, &L.w_down, &L.m_down));
			max_ff = std::max(max_ff, (size_t) L.ff);
		} else if (L.ff_kind == FF_MOE) {
			std::vector<const HostTensor*> up, dn;
			for (int e = 0; e < L.E; e++) {
				const std::string pe = p + "mlp.e" + std::to_string(e) + ".";
				up.push_back(T(pe + "up"));
				dn.push_back(T(pe + "down"));
			}
			XALM_TRY(upload_rows(m, up, W, false, &L.w_up, &L.m_up)); // all experts, one after the other
			XALM_TRY(upload_rows(m, dn, L.ff, false, &L.w_down, &L.m_down));
			XALM_TRY(upload_rows(m, {T(p + "mlp.router")}, W, false, &L.w_router, nullptr));
			XALM_TRY(moe_prepare(W, L.E, 0));
			L.expert_bytes = 2ll * L.ff * W * (m->w_bf16 ? 2 : 4);
			max_pairs = std::max(max_pairs, C * L.top);
			max_moe_hid = std::max(max_moe_hid, C * L.top * L.ff);
			max_tiles = std::max(max_tiles, moe_max_tiles((int) C * L.top, L.E));
		}
		L.bytes = m->weight_bytes - bytes0;
	}
	XALM_TRY(group_norm_prepare(max_norm_width, max_norm_groups));
	for (Layer& L : m->layers) {
		XALM_TRY(tc_register(m, L.m_in, &L.t_in));
		XALM_TRY(tc_register(m, L.m_o, &L.t_o));
		if (L.ff_kind == FF_DENSE) {
			XALM_TRY(tc_register(m, L.m_up, &L.t_up));
			XALM_TRY(tc_register(m, L.m_down, &L.t_down));
		}
		// a mixture whose expert shapes the GEMM takes keeps fp16 tiles per expert for its long passes
		if (L.ff_kind == FF_MOE && m->use_tc && tune("seq_moe_tc") && tc_shape_ok(L.ff, W, L.ff) && tc_shape_ok(W, L.ff, W)) {
			L.t_eup.resize((size_t) L.E);
			L.t_edown.resize((size_t) L.E);
			for (int e = 0; e < L.E; e++) {
				WMat up = L.m_up, dn = L.m_down; // this expert's rows of the stacked matrices
				up.rows = L.ff;
				up.p0 = static_cast<const uint8_t*>(L.m_up.p0) + (size_t) e * L.ff * L.m_up.s0;
				dn.rows = W;
				dn.p0 = static_cast<const uint8_t*>(L.m_down.p0) + (size_t) e * W * L.m_down.s0;
				XALM_TRY(tc_register(m, up, &L.t_eup[(size_t) e]));
				XALM_TRY(tc_register(m, dn, &L.t_edown[(size_t) e]));
			}
			moe_tc = true;
		}
	}
	// what the sequence holds, per layer run
	for (Run& R : m->runs) {
		const Layer& L = m->layers[(size_t) R.layer];
		XALM_TRY(dev_alloc(m, &R.hist, (size_t) 2 * std::max(m->taps - 1, 1) * W, true));
		if (L.mixer == MIX_GLA) XALM_TRY(dev_alloc(m, &R.state, (size_t) L.H * L.d * L.dv, true));
		else {
			XALM_TRY(dev_alloc(m, &R.state, (size_t) L.sH * L.sN * L.sP, true));
			XALM_TRY(dev_alloc(m, &R.conv_hist, (size_t) std::max(L.s_taps - 1, 1) * L.conv_channels(), true));
			uint8_t *kc = nullptr, *vc = nullptr;
			XALM_TRY(dev_alloc(m, &kc, (size_t) m->max_tokens * L.aG * L.ad * kelem, true));
			XALM_TRY(dev_alloc(m, &vc, (size_t) m->max_tokens * L.aG * L.ad * kelem, true));
			R.kc = kc; R.vc = vc;
		}
	}
	m->proj_ld = (int) ((max_proj + 3) / 4 * 4);
	m->part_cap = std::max(4 * 64, 4 * m->chunk); // one-token steps: up to 64 key splits; passes of a prompt: up to 4 per token
	XALM_TRY(dev_alloc(m, &m->x, C * W));
	XALM_TRY(dev_alloc(m, &m->h1, C * W));
	XALM_TRY(dev_alloc(m, &m->h2, C * W));
	XALM_TRY(dev_alloc(m, &m->hn, C * W));
	XALM_TRY(dev_alloc(m, &m->proj, C * m->proj_ld));
	XALM_TRY(dev_alloc(m, &m->att, C * max_att));
	XALM_TRY(dev_alloc(m, &m->yssd, C * max_yssd));
	XALM_TRY(dev_alloc(m, &m->ffh, C * max_ff));
	XALM_TRY(dev_alloc(m, &m->stage_canon, (size_t) 2 * std::max(m->taps - 1, 1) * W, true));
	XALM_TRY(dev_alloc(m, &m->stage_conv, max_conv, true));
	XALM_TRY(dev_alloc(m, &m->part_o, (size_t) m->part_cap * max_hd));
	XALM_TRY(dev_alloc(m, &m->part_ml, (size_t) m->part_cap * 2 * max_h));
	XALM_TRY(dev_alloc(m, &m->tickets, 8 * C, true));
	if (max_pairs) {
		XALM_TRY(dev_alloc(m, &m->moe_idx, max_pairs, true));
		XALM_TRY(dev_alloc(m, &m->moe_wgt, max_pairs, true));
		XALM_TRY(dev_alloc(m, &m->moe_sorted, max_pairs, true));
		XALM_TRY(dev_alloc(m, &m->moe_tiles, (size_t) 3 * max_tiles, true));
		XALM_TRY(dev_alloc(m, &m->moe_ntiles, 1, true));
		XALM_TRY(dev_alloc(m, &m->moe_hid, max_moe_hid));
		XALM_TRY(dev_alloc(m, &m->moe_out, max_pairs * W));
		if (moe_tc) {
			int max_e = 1;
			for (const Layer& L : m->layers) max_e = std::max(max_e, L.E);
			XALM_TRY(dev_alloc(m, &m->moe_off, (size_t) max_e + 1, true));
			XALM_TRY(dev_alloc(m, &m->moe_inv, max_pairs, true));
			XALM_TRY(dev_alloc(m, &m->moe_x, max_pairs * W));
			XALM_CUDA_CHECK(cudaMallocHost(&m->h_off, ((size_t) max_e + 1) * 4));
		}
	}
	return XALM_OK;
}

int release(SeqModel* sm) {
	Kb* m = static_cast<Kb*>(sm);
	for (Run& R : m->runs) {
		const Layer& L = m->layers[(size_t) R.layer];
		XALM_CUDA_CHECK(cudaMemsetAsync(R.hist, 0, (size_t) 2 * std::max(m->taps - 1, 1) * m->width * 4, m->stream));
		if (L.mixer == MIX_GLA) XALM_CUDA_CHECK(cudaMemsetAsync(R.state, 0, (size_t) L.H * L.d * L.dv * 4, m->stream));
		else {
			XALM_CUDA_CHECK(cudaMemsetAsync(R.state, 0, (size_t) L.sH * L.sN * L.sP * 4, m->stream));
			XALM_CUDA_CHECK(cudaMemsetAsync(R.conv_hist, 0, (size_t) std::max(L.s_taps - 1, 1) * L.conv_channels() * 4, m->stream));
		}
	}
	return XALM_OK;
}

// beyond one reading of every matrix: repeated layers read theirs again, a mixture reads only the chosen experts; the visible cache rows,
// the recurrent states read and written
long long active_bytes(SeqModel* sm, long long pos) {
	Kb* m = static_cast<Kb*>(sm);
	const long long kelem = m->precision == XALM_PRECISION_F32 ? 4 : 2, welem = m->w_bf16 ? 2 : 4;
	// the embedding table is read once more, whole, as the head matrix; of the pair table one row
	long long b = (long long) (m->vocab - 1) * m->width * welem - (long long) m->buckets * m->width * welem;
	std::vector<int> seen(m->layers.size(), 0);
	for (const Run& R : m->runs) {
		const Layer& L = m->layers[(size_t) R.layer];
		const long long live = L.bytes - (L.ff_kind == FF_MOE ? (long long) (L.E - L.top) * L.expert_bytes : 0);
		b += seen[(size_t) R.layer]++ ? live : live - L.bytes;
		if (L.mixer == MIX_GLA) b += 2ll * L.H * L.d * L.dv * 4;
		else b += 2ll * L.sH * L.sN * L.sP * 4 + (pos + 1) * 2 * L.aG * L.ad * kelem;
	}
	return b;
}

bool state_buffer(SeqModel* sm, int run, const float** src, size_t* count) {
	Kb* m = static_cast<Kb*>(sm);
	const Run& R = m->runs[(size_t) run];
	const Layer& L = m->layers[(size_t) R.layer];
	*src = R.state;
	*count = L.mixer == MIX_GLA ? (size_t) L.H * L.d * L.dv : (size_t) L.sH * L.sN * L.sP;
	return true;
}

void destroy(SeqModel* sm) {
	Kb* m = static_cast<Kb*>(sm);
	for (Layer& L : m->layers) {
		for (TcWeight* t : {&L.t_in, &L.t_o, &L.t_up, &L.t_down}) tc_weight_free(t);
		for (TcWeight& t : L.t_eup) tc_weight_free(&t);
		for (TcWeight& t : L.t_edown) tc_weight_free(&t);
	}
	if (m->h_off) cudaFreeHost(m->h_off);
	delete m;
}

const SeqHooks kubolorn_hooks = {parse_config, finalize, enqueue_pass, release, active_bytes, state_buffer, destroy};
extern const ModelFamily kubolorn_family;
int create(const char* json, int device, int max_tokens, int precision, xalm_cuda_model** out) {
	return seq_create<Kb>(&kubolorn_family, &kubolorn_hooks, json, device, max_tokens, precision, out);
}
const ModelFamily kubolorn_family = seq_family_table("Kubolorn", create);
const FamilyRegistrar kubolorn_registrar(&kubolorn_family);

} // namespace
} // namespace xalm
