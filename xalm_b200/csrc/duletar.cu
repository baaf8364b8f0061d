// duletar.cu — the Duletar family of the model registry (family.h): a pre-norm decoder described by a config.json whose layers each
// carry ONE token mixer, chosen per layer, and an optional feed-forward:
//
//   mixer "latent_attention"    softmax attention whose keys and values are expanded per head from a low-rank latent c = rmsnorm(W_dkv h);
//                               queries pass a latent of their own; each head has d plain and r rotated query/key entries, the rotated
//                               key part is one vector shared by all heads; causal, no window
//   mixer "latent_attention_2"  the same without positions, with a sigmoid output gate; a layer may read another layer's latents
//                               ("kv_from") through expansions of its own
//   mixer "retention"           linear attention with one fixed decay per head: S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t, rotary
//                               positions on q and k, o over its root mean square, silu output gate
//   feed-forward                dense W_down relu(W_up h)^2, or a mixture of clamped gated experts: softmax scores over all experts, groups
//                               scored by their best expert limit the choice, weights = chosen scores over their sum
//
// x <- x + mixer(rmsnorm(x) w1), x <- x + ff(rmsnorm(x) w2); the embedding row is scaled; logits = cap * tanh(head . rmsnorm(x) / cap).
//
// The step function, graph replay of one-token steps, uploads, release and the C entry points are the shared sequence engine's
// (seq_family.cuh).  Per pass and layer here:
//     latent attention: norm -> rows product [dq | dkv | gate] -> latent_post (latent norms, rotated key, cache row) -> rows product [uq]
//                       -> batched per-head product with uk^T (queries into the latent) + rope_heads (rotated query part) -> swa_attn /
//                       swa_tile with ONE key/value head reading the cache rows in place -> batched per-head product with uv (gate fused)
//                       -> rows product [o] with the residual add fused
//     retention:        norm -> rows product [q | k | v | gate] -> rope_heads in place -> hgrn2 kernels in their fixed-decay mode (norm and
//                       gate fused) -> rows product [o] + residual
//     dense ff:         norm -> rows product [up, relu^2 fused] -> rows product [down] + residual
//     experts:          norm -> moe_router -> moe_sort -> moe_gemm [gate | up, clamped GLU fused] -> moe_gemm [down] -> moe_combine (+ residual)
//
// Cache / state manager: a latent-attention layer keeps ONE row of kv_rank + rot_dim elements per position (the normed latent and the
// rotated shared key), nothing per head; a layer with kv_from keeps nothing and reads the other layer's rows.  A retention layer keeps
// its fp32 state (heads x dim x vdim).  release() zeroes the states; cache rows need no clearing, a sequence only reads positions it wrote.
//
// Precision: the residual stream, norms, rotation angles, scores, softmax, router, the recurrence with its state, gates and every sum are
// fp32 in both modes.  XALM_PRECISION_BF16 keeps matrices and the latent cache in bf16 and sends dense products of long passes through
// the tcgen05 GEMM (fp16 operands, fp32 accumulation); XALM_PRECISION_F32 widens both and uses the fp32 FMA kernels only.
#include "seq_family.cuh"

#include "latent_ops.cuh"
#include "moe_ops.cuh"

namespace xalm {
namespace {

using namespace mix;
using namespace seq;

enum { MIX_LATENT = 0, MIX_LATENT_GATED = 1, MIX_RETENTION = 2 };
enum { FF_NONE = 0, FF_DENSE = 1, FF_MOE = 2 };

struct Layer {
	int mixer = MIX_LATENT, ff_kind = FF_NONE;
	int H = 0, d = 0, dv = 0;
	// latent attention: r rotated entries per head, R / Rq latent sizes of keys+values / queries
	int r = 0, R = 0, Rq = 0, kv_from = -1;
	float scale = 1.f;
	float *dq_norm = nullptr, *dkv_norm = nullptr;
	void* cache = nullptr; // (max_tokens, cache_ld): this layer's rows, or the rows of the layer it reads
	int cache_ld = 0;
	void *w_uq = nullptr, *w_ukT = nullptr, *w_uv = nullptr;
	WMat m_uq;
	TcWeight t_uq;
	// retention
	int rot_dims = 0;
	std::vector<float> decay_host;
	float *decay = nullptr, *state = nullptr;
	// both
	std::vector<float> freq_host;
	float* freq = nullptr;
	int off_a = 0, off_b = 0, off_g = 0, n_in = 0; // columns of the stacked input projection: [dq | dkv | g] or [q | k | v | g]
	// feed-forward
	int ff = 0, E = 0, top = 0, n_groups = 0, keep_groups = 0;
	float limit = 0.f;
	void *w_in = nullptr, *w_o = nullptr, *w_up = nullptr, *w_down = nullptr, *w_router = nullptr;
	WMat m_in, m_o, m_up, m_down;
	TcWeight t_in, t_o, t_up, t_down;
	std::vector<TcWeight> t_egu, t_edown; // per expert, when the mixture's long passes run on the tensor cores
	float *norm1 = nullptr, *norm2 = nullptr;
};

struct DuletarModel : SeqModel {
	float embed_scale = 1.f, logit_cap = 0.f;
	std::vector<Layer> layers;
	// one pass
	float *x = nullptr, *hn = nullptr, *proj = nullptr, *cq = nullptr, *q = nullptr, *qabs = nullptr, *olat = nullptr, *att = nullptr, *ffh = nullptr;
	int proj_ld = 4;
	float *part_o = nullptr, *part_ml = nullptr;
	unsigned* tickets = nullptr;
	int part_cap = 0;
	int *moe_idx = nullptr, *moe_sorted = nullptr, *moe_tiles = nullptr, *moe_ntiles = nullptr;
	float *moe_wgt = nullptr, *moe_hid = nullptr, *moe_out = nullptr;
	int *moe_off = nullptr, *moe_inv = nullptr, *h_off = nullptr;
	float* moe_x = nullptr;
};
typedef DuletarModel Du;

std::vector<float> rotary_frequencies(double base, int dims) { // f_i = base^(-2i/dims)
	std::vector<float> f((size_t) dims / 2);
	for (int i = 0; i < dims / 2; i++) f[(size_t) i] = (float) pow(base, -2.0 * i / dims);
	return f;
}

// ---- config.json ------------------------------------------------------------------------------------------------------------------
int parse_config(SeqModel* sm, const char* json) {
	Du* m = static_cast<Du*>(sm);
	try {
		const xjson::Value c = xjson::Parser::parse(json, strlen(json));
		m->vocab = geti(c, "vocab");
		m->width = geti(c, "width");
		if (const xjson::Value* nv = c.find("norm"))
			if (const xjson::Value* e = nv->find("eps")) m->eps = (float) e->num;
		if (const xjson::Value* ev = c.find("embedding"); ev && ev->kind == xjson::Value::Obj && ev->contains("scale")) m->embed_scale = (float) getf(*ev, "scale");
		if (const xjson::Value* lc = c.find("logit_softcap"); lc && lc->kind == xjson::Value::Number) m->logit_cap = (float) lc->num;
		if (m->vocab <= 0 || m->width <= 0) return set_error(XALM_ERR_INVALID, "config: vocab / width must be positive");
		const int W = m->width;
		expect(m, "embed", {m->vocab, W}, true);
		const xjson::Value& layers = c.at("layers");
		if (layers.kind != xjson::Value::Array || layers.arr.empty()) return set_error(XALM_ERR_INVALID, "config: no layers");
		for (size_t li = 0; li < layers.arr.size(); li++) {
			const xjson::Value& lv = layers.arr[li];
			const std::string type = lv.at("type").str;
			Layer L;
			if (type == "latent_attention") L.mixer = MIX_LATENT;
			else if (type == "latent_attention_2") L.mixer = MIX_LATENT_GATED;
			else if (type == "retention") L.mixer = MIX_RETENTION;
			else return set_error(XALM_ERR_UNSUPPORTED, "config: layer %zu has mixer type '%s' (this family runs 'latent_attention', 'latent_attention_2' and 'retention')", li, type.c_str());
			const xjson::Value& mx = lv.at("mixer");
			L.H = geti(mx, "heads");
			L.d = geti(mx, "dim");
			L.dv = mx.contains("vdim") ? geti(mx, "vdim") : L.d;
			if (L.H <= 0 || L.d <= 0 || L.dv <= 0) return set_error(XALM_ERR_INVALID, "config: layer %zu: bad mixer sizes", li);
			const std::string p = "l" + std::to_string(li) + ".";
			const int H = L.H, d = L.d, dv = L.dv;
			const xjson::Value* rt = mx.find("rot");
			if (rt && rt->kind != xjson::Value::Obj) rt = nullptr;
			expect(m, p + "norm1", {W}, false);
			if (L.mixer == MIX_RETENTION) {
				const xjson::Value& dc = mx.at("decay");
				if (dc.kind != xjson::Value::Array || (int) dc.arr.size() != H) return set_error(XALM_ERR_INVALID, "config: layer %zu: 'decay' lists one value per head", li);
				for (const xjson::Value& v : dc.arr) L.decay_host.push_back((float) v.num);
				if (rt) {
					L.rot_dims = geti(*rt, "dims");
					if (L.rot_dims < 0 || L.rot_dims > d || L.rot_dims % 2) return set_error(XALM_ERR_INVALID, "config: layer %zu: %d rotary dimensions in a head of %d", li, L.rot_dims, d);
					if (L.rot_dims) L.freq_host = rotary_frequencies(getf(*rt, "base"), L.rot_dims);
				}
				expect(m, p + "mix.q", {H * d, W}, true);
				expect(m, p + "mix.k", {H * d, W}, true);
				expect(m, p + "mix.v", {H * dv, W}, true);
				expect(m, p + "mix.g", {H * dv, W}, true);
			} else {
				L.R = geti(mx, "kv_rank");
				L.Rq = geti(mx, "q_rank");
				L.scale = mx.contains("scale") ? (float) getf(mx, "scale") : 1.f / sqrtf((float) d);
				if (L.mixer == MIX_LATENT) {
					L.r = mx.contains("rot_dim") ? geti(mx, "rot_dim") : 0;
					if (L.r < 0 || L.r % 2) return set_error(XALM_ERR_INVALID, "config: layer %zu: rot_dim %d", li, L.r);
					if (L.r) {
						if (!rt) return set_error(XALM_ERR_INVALID, "config: layer %zu: rot_dim without 'rot'", li);
						const int dims = rt->contains("dims") ? geti(*rt, "dims") : L.r;
						if (dims != L.r) return set_error(XALM_ERR_INVALID, "config: layer %zu: rot.dims %d differs from rot_dim %d", li, dims, L.r);
						L.freq_host = rotary_frequencies(getf(*rt, "base"), L.r);
					}
				}
				if (L.R <= 0 || L.Rq <= 0) return set_error(XALM_ERR_INVALID, "config: layer %zu: latent sizes", li);
				if (const xjson::Value* kf = mx.find("kv_from"); kf && kf->kind == xjson::Value::Number) {
					if (L.mixer != MIX_LATENT_GATED) return set_error(XALM_ERR_UNSUPPORTED, "config: layer %zu: kv_from on a rotary latent attention", li);
					L.kv_from = (int) kf->num;
					if (L.kv_from < 0 || L.kv_from >= (int) li) return set_error(XALM_ERR_INVALID, "config: layer %zu: kv_from %d is not an earlier layer", li, L.kv_from);
					const Layer& J = m->layers[(size_t) L.kv_from];
					if (J.mixer == MIX_RETENTION || J.kv_from >= 0 || J.R != L.R)
						return set_error(XALM_ERR_INVALID, "config: layer %zu: layer %d has no latents of %d of its own", li, L.kv_from, L.R);
				}
				expect(m, p + "mix.dq", {L.Rq, W}, true);
				expect(m, p + "mix.dq.norm", {L.Rq}, false);
				expect(m, p + "mix.uq", {H * (d + L.r), L.Rq}, true);
				if (L.kv_from < 0) {
					expect(m, p + "mix.dkv", {L.R + L.r, W}, true);
					expect(m, p + "mix.dkv.norm", {L.R}, false);
				}
				expect(m, p + "mix.uk", {H * d, L.R}, true);
				expect(m, p + "mix.uv", {H * dv, L.R}, true);
				if (L.mixer == MIX_LATENT_GATED) expect(m, p + "mix.g", {H * dv, W}, true);
			}
			expect(m, p + "mix.o", {W, H * dv}, true);
			const xjson::Value* mlp = lv.find("mlp");
			if (mlp && mlp->kind == xjson::Value::Obj) {
				const std::string kind = mlp->contains("kind") ? mlp->at("kind").str : "dense";
				expect(m, p + "norm2", {W}, false);
				if (kind == "dense") {
					L.ff_kind = FF_DENSE;
					L.ff = geti(*mlp, "ff");
					if (L.ff <= 0) return set_error(XALM_ERR_INVALID, "config: layer %zu: ff", li);
					expect(m, p + "mlp.up", {L.ff, W}, true);
					expect(m, p + "mlp.down", {W, L.ff}, true);
				} else if (kind == "moe") {
					L.ff_kind = FF_MOE;
					const xjson::Value& ex = mlp->at("expert");
					L.ff = geti(ex, "ff");
					L.limit = (float) getf(ex, "limit");
					const xjson::Value& r = mlp->at("router");
					L.E = geti(r, "experts");
					L.top = geti(r, "top");
					if (const xjson::Value* g = r.find("groups"); g && g->kind == xjson::Value::Obj) {
						L.n_groups = geti(*g, "count");
						L.keep_groups = geti(*g, "keep");
					}
					if (L.ff <= 0 || L.E <= 0 || L.top <= 0 || L.top > L.E) return set_error(XALM_ERR_INVALID, "config: layer %zu: %d of %d experts of %d", li, L.top, L.E, L.ff);
					if (L.n_groups > 1 && (L.E % L.n_groups || L.keep_groups <= 0 || L.keep_groups > L.n_groups || L.keep_groups * (L.E / L.n_groups) < L.top))
						return set_error(XALM_ERR_INVALID, "config: layer %zu: %d expert groups with %d kept cannot hold %d of %d experts", li, L.n_groups, L.keep_groups, L.top, L.E);
					for (int e = 0; e < L.E; e++) {
						const std::string pe = p + "mlp.e" + std::to_string(e) + ".";
						expect(m, pe + "gate", {L.ff, W}, true);
						expect(m, pe + "up", {L.ff, W}, true);
						expect(m, pe + "down", {W, L.ff}, true);
					}
					expect(m, p + "mlp.router", {L.E, W}, true);
				} else return set_error(XALM_ERR_UNSUPPORTED, "config: layer %zu has feed-forward kind '%s'", li, kind.c_str());
			}
			m->layers.push_back(std::move(L));
		}
		m->n_layers = (int) m->layers.size();
		expect(m, "final.norm", {W}, false);
		expect(m, "head", {m->vocab, W}, true);
	} catch (const std::exception& e) {
		return set_error(XALM_ERR_INVALID, "config.json: %s", e.what());
	}
	return XALM_OK;
}

// ---- the kernels of one pass ----------------------------------------------------------------------------------------------------------
RowsEpi residual_epi(Du* m) { // x <- x + product: the single-stream case of the hyper-connection write
	RowsEpi e;
	e.kind = EPI_HC;
	e.xs = m->x;
	e.S = 1;
	e.stream_stride = (size_t) m->chunk * m->width;
	return e;
}

int enqueue_latent(Du* m, const Layer& L, int n, int* nl) {
	cudaStream_t s = m->stream;
	const int H = L.H, d = L.d, r = L.r, dv = L.dv, R = L.R, Rq = L.Rq;
	const bool f32 = m->precision == XALM_PRECISION_F32;
	LatentPostArgs pa = {};
	pa.proj = m->proj; pa.ld = m->proj_ld;
	pa.q_off = 0; pa.q_rank = Rq; pa.q_norm = L.dq_norm; pa.cq = m->cq; pa.ldc = Rq;
	pa.kv_off = L.off_a; pa.kv_rank = L.kv_from < 0 ? R : 0; pa.rot = r; pa.kv_norm = L.dkv_norm; pa.freq = L.freq;
	pa.eps = m->eps; pa.cache = L.cache; pa.cache_f32 = f32; pa.ring = m->max_tokens; pa.step = m->d_step;
	XALM_TRY(launch_latent_post(pa, n, s));
	(*nl)++;
	RowsEpi est;
	est.kind = EPI_STORE; est.out = m->q; est.ldo = H * (d + r);
	XALM_TRY(rows_product(m, m->cq, Rq, L.w_uq, &L.t_uq, n, H * (d + r), Rq, est, nl));
	// queries into the latent, head by head: qabs[h] = [uk_h^T q_h | rotated q_h]
	RowsEpi eb;
	eb.kind = EPI_STORE; eb.out = m->qabs; eb.ldo = H * (R + r);
	eb.batch_a = d + r; eb.batch_w = (size_t) R * d; eb.batch_o = R + r;
	XALM_TRY(launch_rows(m->q, H * (d + r), L.w_ukT, m->w_bf16, n, R, d, eb, s, H));
	(*nl)++;
	if (r) {
		RopeHeadsArgs ra = {};
		ra.src = m->q; ra.lds = H * (d + r); ra.src_off = d; ra.src_stride = d + r;
		ra.dst = m->qabs; ra.ldd = H * (R + r); ra.dst_off = R; ra.dst_stride = R + r;
		ra.heads = H; ra.n = r; ra.rot_half = r / 2; ra.freq = L.freq; ra.step = m->d_step;
		XALM_TRY(launch_rope_heads(ra, n, s));
		(*nl)++;
	}
	SwaArgs sa = {};
	sa.q = m->qabs; sa.ldq = H * (R + r); sa.q_off = 0;
	sa.kc = L.cache; sa.vc = L.cache; sa.ldk = L.cache_ld; sa.ldv = L.cache_ld;
	sa.ring = m->max_tokens; sa.keep_first = 0;
	sa.H = H; sa.G = 1; sa.d = R + r; sa.dv = R;
	sa.window = 0x7fffffff; sa.scale = L.scale;
	sa.step = m->d_step; sa.out = m->olat;
	sa.n_splits = 0;
	sa.part_o = m->part_o; sa.part_ml = m->part_ml; sa.part_cap = m->part_cap; sa.tickets = m->tickets;
	int swa_launches = 1;
	XALM_TRY(launch_swa(sa, n, f32, s, &swa_launches));
	*nl += swa_launches;
	// values out of the latent, head by head, with the output gate
	RowsEpi ev;
	ev.kind = EPI_STORE; ev.out = m->att; ev.ldo = H * dv;
	ev.batch_a = R; ev.batch_w = (size_t) dv * R; ev.batch_o = dv;
	if (L.mixer == MIX_LATENT_GATED) { ev.mul = m->proj + L.off_g; ev.ldm = m->proj_ld; ev.mul_act = ACT_SIGMOID; }
	XALM_TRY(launch_rows(m->olat, H * R, L.w_uv, m->w_bf16, n, dv, R, ev, s, H));
	(*nl)++;
	return XALM_OK;
}

int enqueue_retention(Du* m, const Layer& L, int n, int* nl) {
	cudaStream_t s = m->stream;
	const int H = L.H, d = L.d, dv = L.dv;
	if (L.rot_dims) {
		RopeHeadsArgs ra = {};
		ra.src = m->proj; ra.dst = m->proj; ra.lds = ra.ldd = m->proj_ld; ra.src_off = ra.dst_off = 0; ra.src_stride = ra.dst_stride = d;
		ra.heads = 2 * H; ra.n = d; ra.rot_half = L.rot_dims / 2; ra.freq = L.freq; ra.step = m->d_step; // q heads, then k heads
		XALM_TRY(launch_rope_heads(ra, n, s));
		(*nl)++;
	}
	Hgrn2Args ha = {};
	ha.proj = m->proj; ha.ld = m->proj_ld; ha.q_off = 0; ha.k_off = L.off_a; ha.v_off = L.off_b;
	ha.H = H; ha.d = d; ha.dv = dv;
	ha.decay = L.decay; ha.k_scale = 1.f / sqrtf((float) d);
	ha.norm_plain = 1; ha.eps = m->eps;
	ha.gate = m->proj; ha.ldg = m->proj_ld; ha.g_off = L.off_g;
	ha.state = L.state; ha.step = m->d_step; ha.out = m->att; ha.max_rows = m->chunk;
	XALM_TRY(launch_hgrn2(ha, s));
	(*nl)++;
	return XALM_OK;
}

int enqueue_experts(Du* m, const Layer& L, int n, int* nl) {
	cudaStream_t s = m->stream;
	const int W = m->width;
	MoeRouteArgs ra = {};
	ra.h = m->hn; ra.ldh = W; ra.w = L.w_router; ra.w_bf16 = m->w_bf16;
	ra.E = L.E; ra.top = L.top; ra.K = W; ra.n_groups = L.n_groups; ra.keep_groups = L.keep_groups;
	ra.idx = m->moe_idx; ra.wgt = m->moe_wgt; ra.step = m->d_step;
	ra.score_kind = MOE_SCORE_SOFTMAX; ra.group_kind = MOE_GROUP_MAX; ra.renormalise = 1; ra.renorm_eps = 1e-20f;
	XALM_TRY(launch_moe_router(ra, n, s));
	(*nl)++;
	const bool on_tc = m->use_tc && !L.t_egu.empty() && n >= m->tc_min_rows;
	const bool tiled = on_tc || n * L.top > MOE_MATVEC_PAIRS; // steps of a few tokens run one matvec per (token, slot) pair and need no tile list
	if (tiled) {
		MoeSortArgs so = {m->moe_idx, L.top, L.E, m->d_step, m->moe_sorted, m->moe_tiles, m->moe_ntiles, m->moe_off, m->moe_inv};
		XALM_TRY(launch_moe_sort(so, s));
		(*nl)++;
	}
	RowsEpi eg;
	eg.kind = EPI_GLU; eg.glu_act = GLU_CLAMPED; eg.limit = L.limit; eg.alpha = 1.702f; eg.ldo = L.ff;
	if (on_tc) {
		// Long passes of the 16-bit mode: each expert's rows, gathered one after the other, go through the tcgen05 GEMM on that expert's
		// resident fp16 tiles.  How many rows each expert got is read back first (one small copy and a wait per mixture layer and pass).
		XALM_CUDA_CHECK(cudaMemcpyAsync(m->h_off, m->moe_off, (size_t) (L.E + 1) * 4, cudaMemcpyDeviceToHost, s));
		moe_gather_kernel<<<n * L.top, 256, 0, s>>>(m->hn, W, L.top, m->moe_sorted, m->d_step, L.top, W, m->moe_x);
		XALM_SEQ_LAUNCH_CHECK("moe_gather");
		XALM_CUDA_CHECK(cudaStreamSynchronize(s));
		for (int e = 0; e < L.E; e++) {
			const int at = m->h_off[e], cnt = m->h_off[e + 1] - at;
			if (cnt <= 0) continue;
			XALM_TRY(tc_gemm(L.t_egu[(size_t) e], m->moe_x + (size_t) at * W, cnt, m->tc_out, 2 * L.ff, m->a_hi, m->a_lo, s));
			eg.out = m->moe_hid + (size_t) at * L.ff;
			XALM_TRY(launch_rows_epilogue(m->tc_out, 2 * L.ff, cnt, 2 * L.ff, eg, s));
			XALM_TRY(tc_gemm(L.t_edown[(size_t) e], m->moe_hid + (size_t) at * L.ff, cnt, m->moe_out + (size_t) at * W, W, m->a_hi, m->a_lo, s));
			*nl += 5;
		}
	} else {
		MoeGemmArgs ga = {};
		ga.A = m->hn; ga.lda = W; ga.a_div = L.top; ga.W = L.w_up; ga.N = 2 * L.ff; ga.K = W;
		ga.sorted = m->moe_sorted; ga.tiles = m->moe_tiles; ga.n_tiles = m->moe_ntiles;
		ga.idx = m->moe_idx; ga.step = m->d_step; ga.top = L.top;
		ga.e = eg; ga.e.out = m->moe_hid;
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
	Du* m = static_cast<Du*>(sm);
	cudaStream_t s = m->stream;
	const int W = m->width;
	const size_t hs = (size_t) m->chunk * W;
	if (m->w_bf16) embed_streams_kernel<__nv_bfloat16><<<n, norm_threads(W), 0, s>>>((const __nv_bfloat16*) m->embed, m->d_tokens, W, 1, hs, m->x, m->embed_scale);
	else embed_streams_kernel<float><<<n, norm_threads(W), 0, s>>>((const float*) m->embed, m->d_tokens, W, 1, hs, m->x, m->embed_scale);
	XALM_SEQ_LAUNCH_CHECK("embed");
	for (size_t li = 0; li < m->layers.size(); li++) {
		const Layer& L = m->layers[li];
		XALM_TRY(launch_hc_norm(m->x, 1, hs, nullptr, L.norm1, 0, m->eps, W, m->hn, nullptr, n, s));
		(*nl)++;
		RowsEpi est;
		est.kind = EPI_STORE; est.out = m->proj; est.ldo = m->proj_ld;
		XALM_TRY(rows_product(m, m->hn, W, L.w_in, &L.t_in, n, L.n_in, W, est, nl));
		if (L.mixer == MIX_RETENTION) XALM_TRY(enqueue_retention(m, L, n, nl));
		else XALM_TRY(enqueue_latent(m, L, n, nl));
		XALM_TRY(rows_product(m, m->att, L.H * L.dv, L.w_o, &L.t_o, n, W, L.H * L.dv, residual_epi(m), nl));
		if (L.ff_kind != FF_NONE) {
			XALM_TRY(launch_hc_norm(m->x, 1, hs, nullptr, L.norm2, 0, m->eps, W, m->hn, nullptr, n, s));
			(*nl)++;
		}
		if (L.ff_kind == FF_DENSE) {
			RowsEpi ea;
			ea.kind = EPI_ACT; ea.act = ACT_RELU_SQUARED; ea.out = m->ffh; ea.ldo = L.ff;
			XALM_TRY(rows_product(m, m->hn, W, L.w_up, &L.t_up, n, L.ff, W, ea, nl));
			XALM_TRY(rows_product(m, m->ffh, L.ff, L.w_down, &L.t_down, n, W, L.ff, residual_epi(m), nl));
		} else if (L.ff_kind == FF_MOE) XALM_TRY(enqueue_experts(m, L, n, nl));
		if (m->keep_layers) XALM_CUDA_CHECK(cudaMemcpyAsync(m->layer_sums + li * hs, m->x, (size_t) n * W * 4, cudaMemcpyDeviceToDevice, s));
	}
	if (want) {
		const int rows = want == 2 ? n : 1, first = want == 2 ? 0 : n - 1;
		XALM_TRY(launch_hc_norm(m->x + (size_t) first * W, 1, hs, nullptr, m->final_norm, 0, m->eps, W, m->hn, nullptr, rows, s));
		(*nl)++;
		RowsEpi eh;
		eh.kind = EPI_STORE; eh.out = m->logits; eh.ldo = m->vocab; eh.cap = m->logit_cap;
		XALM_TRY(rows_product(m, m->hn, W, m->w_head, &m->t_head, rows, m->vocab, W, eh, nl));
	}
	return XALM_OK;
}

// ---- device layouts, cache, state, pass buffers ---------------------------------------------------------------------------------------
// uk (H * d, R) as H matrices (R, d): row j of head h holds column j of that head's rows, so that q_h -> uk_h^T q_h is a rows product
int upload_transposed_heads(Du* m, const HostTensor* uk, int H, int d, int R, void** dst) {
	HostTensor t;
	t.shape = {H * R, d};
	t.v.resize((size_t) H * R * d);
	for (int h = 0; h < H; h++)
		for (int i = 0; i < d; i++)
			for (int j = 0; j < R; j++) t.v[((size_t) h * R + j) * d + i] = uk->v[((size_t) h * d + i) * R + j];
	return upload_rows(m, {&t}, d, false, dst, nullptr);
}

int finalize(SeqModel* sm) {
	Du* m = static_cast<Du*>(sm);
	const int W = m->width;
	const size_t C = (size_t) m->chunk;
	auto T = [&](const std::string& n) { return tensor_or_null(m, n); };
	size_t max_in = 4, max_cq = 1, max_q = 1, max_qabs = 1, max_olat = 1, max_att = 1, max_ff = 1, max_h = 1, max_pairs = 0, max_moe_hid = 0;
	int max_tiles = 1;
	bool moe_tc = false;
	const size_t kelem = m->precision == XALM_PRECISION_F32 ? 4 : 2;
	for (size_t li = 0; li < m->layers.size(); li++) {
		Layer& L = m->layers[li];
		const std::string p = "l" + std::to_string(li) + ".";
		const int H = L.H, d = L.d, dv = L.dv, r = L.r, R = L.R, Rq = L.Rq;
		XALM_TRY(upload_vec(m, p + "norm1", &L.norm1));
		if (!L.freq_host.empty()) XALM_TRY(upload_floats(m, L.freq_host.data(), L.freq_host.size(), &L.freq));
		if (L.mixer == MIX_RETENTION) {
			L.off_a = H * d; L.off_b = 2 * H * d; L.off_g = L.off_b + H * dv; L.n_in = L.off_g + H * dv;
			XALM_TRY(upload_rows(m, {T(p + "mix.q"), T(p + "mix.k"), T(p + "mix.v"), T(p + "mix.g")}, W, false, &L.w_in, &L.m_in));
			XALM_TRY(upload_floats(m, L.decay_host.data(), L.decay_host.size(), &L.decay));
			XALM_TRY(dev_alloc(m, &L.state, (size_t) H * d * dv, true));
			if (!hgrn2_cols_ok(d, dv, m->chunk) && hgrn2_smem_bytes(d, dv) > 200 * 1024)
				return set_error(XALM_ERR_UNSUPPORTED, "layer %zu: a retention state of %d x %d per head", li, d, dv);
			XALM_TRY(hgrn2_prepare(d, dv));
		} else {
			const bool own = L.kv_from < 0;
			L.off_a = Rq; L.off_g = Rq + (own ? R + r : 0);
			L.n_in = L.off_g + (L.mixer == MIX_LATENT_GATED ? H * dv : 0);
			XALM_TRY(upload_rows(m, {T(p + "mix.dq"), own ? T(p + "mix.dkv") : nullptr, L.mixer == MIX_LATENT_GATED ? T(p + "mix.g") : nullptr}, W, false, &L.w_in, &L.m_in));
			XALM_TRY(upload_vec(m, p + "mix.dq.norm", &L.dq_norm));
			XALM_TRY(upload_rows(m, {T(p + "mix.uq")}, Rq, false, &L.w_uq, &L.m_uq));
			XALM_TRY(upload_transposed_heads(m, T(p + "mix.uk"), H, d, R, &L.w_ukT));
			XALM_TRY(upload_rows(m, {T(p + "mix.uv")}, R, false, &L.w_uv, nullptr));
			if (own) {
				XALM_TRY(upload_vec(m, p + "mix.dkv.norm", &L.dkv_norm));
				L.cache_ld = R + r;
				uint8_t* cache = nullptr;
				XALM_TRY(dev_alloc(m, &cache, (size_t) m->max_tokens * L.cache_ld * kelem, true));
				L.cache = cache;
			} else {
				L.cache = m->layers[(size_t) L.kv_from].cache;
				L.cache_ld = m->layers[(size_t) L.kv_from].cache_ld;
			}
			// the attention sees one key/value head of R + r (values: R)
			if (!swa_pick_tq(H, 1, R + r, R, m->chunk) && swa_smem_bytes(H, R + r, R) > 200 * 1024)
				return set_error(XALM_ERR_UNSUPPORTED, "layer %zu: %d heads over a latent of %d + %d need %zu bytes of shared memory", li, H, R, r, swa_smem_bytes(H, R + r, R));
			XALM_TRY(swa_prepare(H, R + r, R));
			max_cq = std::max(max_cq, (size_t) Rq);
			max_q = std::max(max_q, (size_t) H * (d + r));
			max_qabs = std::max(max_qabs, (size_t) H * (R + r));
			max_olat = std::max(max_olat, (size_t) H * R);
			max_h = std::max(max_h, (size_t) H);
		}
		XALM_TRY(upload_rows(m, {T(p + "mix.o")}, H * dv, false, &L.w_o, &L.m_o));
		max_in = std::max(max_in, (size_t) L.n_in);
		max_att = std::max(max_att, (size_t) H * dv);
		if (L.ff_kind != FF_NONE) XALM_TRY(upload_vec(m, p + "norm2", &L.norm2));
		if (L.ff_kind == FF_DENSE) {
			XALM_TRY(upload_rows(m, {T(p + "mlp.up")}, W, false, &L.w_up, &L.m_up));
			XALM_TRY(upload_rows(m, {T(p + "mlp.down")}, L.ff, false, &L.w_down, &L.m_down));
			max_ff = std::max(max_ff, (size_t) L.ff);
		} else if (L.ff_kind == FF_MOE) {
			std::vector<const HostTensor*> gu, dn;
			for (int e = 0; e < L.E; e++) {
				const std::string pe = p + "mlp.e" + std::to_string(e) + ".";
				gu.push_back(T(pe + "gate"));
				gu.push_back(T(pe + "up"));
				dn.push_back(T(pe + "down"));
			}
			XALM_TRY(upload_rows(m, gu, W, true, &L.w_up, &L.m_up)); // all experts, one after the other, gate / up rows alternating
			XALM_TRY(upload_rows(m, dn, L.ff, false, &L.w_down, &L.m_down));
			XALM_TRY(upload_rows(m, {T(p + "mlp.router")}, W, false, &L.w_router, nullptr));
			XALM_TRY(moe_prepare(W, L.E, L.n_groups));
			max_pairs = std::max(max_pairs, C * L.top);
			max_moe_hid = std::max(max_moe_hid, C * L.top * L.ff);
			max_tiles = std::max(max_tiles, moe_max_tiles((int) C * L.top, L.E));
		}
	}
	XALM_TRY(hc_norm_prepare(W));
	for (Layer& L : m->layers) {
		XALM_TRY(tc_register(m, L.m_in, &L.t_in));
		XALM_TRY(tc_register(m, L.m_o, &L.t_o));
		if (L.mixer != MIX_RETENTION) XALM_TRY(tc_register(m, L.m_uq, &L.t_uq));
		if (L.ff_kind == FF_DENSE) {
			XALM_TRY(tc_register(m, L.m_up, &L.t_up));
			XALM_TRY(tc_register(m, L.m_down, &L.t_down));
		}
		// a mixture whose expert shapes the GEMM takes keeps fp16 tiles per expert for its long passes
		if (L.ff_kind == FF_MOE && m->use_tc && tune("seq_moe_tc") && tc_shape_ok(2 * L.ff, W, 2 * L.ff) && tc_shape_ok(W, L.ff, W)) {
			L.t_egu.resize((size_t) L.E);
			L.t_edown.resize((size_t) L.E);
			for (int e = 0; e < L.E; e++) {
				WMat gu = L.m_up, dn = L.m_down; // this expert's rows of the stacked matrices
				gu.rows = 2 * L.ff;
				gu.p0 = static_cast<const uint8_t*>(L.m_up.p0) + (size_t) e * 2 * L.ff * L.m_up.s0;
				dn.rows = W;
				dn.p0 = static_cast<const uint8_t*>(L.m_down.p0) + (size_t) e * W * L.m_down.s0;
				XALM_TRY(tc_register(m, gu, &L.t_egu[(size_t) e]));
				XALM_TRY(tc_register(m, dn, &L.t_edown[(size_t) e]));
			}
			moe_tc = true;
		}
	}
	m->proj_ld = (int) ((max_in + 3) / 4 * 4);
	m->part_cap = std::max(4 * 64, 4 * m->chunk); // one-token steps: up to 64 key splits; passes of a prompt: up to 4 per token
	XALM_TRY(dev_alloc(m, &m->x, C * W));
	XALM_TRY(dev_alloc(m, &m->hn, C * W));
	XALM_TRY(dev_alloc(m, &m->proj, C * m->proj_ld));
	XALM_TRY(dev_alloc(m, &m->cq, C * max_cq));
	XALM_TRY(dev_alloc(m, &m->q, C * max_q));
	XALM_TRY(dev_alloc(m, &m->qabs, C * max_qabs));
	XALM_TRY(dev_alloc(m, &m->olat, C * max_olat));
	XALM_TRY(dev_alloc(m, &m->att, C * max_att));
	XALM_TRY(dev_alloc(m, &m->ffh, C * max_ff));
	XALM_TRY(dev_alloc(m, &m->part_o, (size_t) m->part_cap * max_olat));
	XALM_TRY(dev_alloc(m, &m->part_ml, (size_t) m->part_cap * 2 * max_h));
	XALM_TRY(dev_alloc(m, &m->tickets, 8 * C, true)); // the heads of a layer may run in up to 8 launches, each with counters of its own
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
	Du* m = static_cast<Du*>(sm);
	for (Layer& L : m->layers)
		if (L.mixer == MIX_RETENTION) XALM_CUDA_CHECK(cudaMemsetAsync(L.state, 0, (size_t) L.H * L.d * L.dv * 4, m->stream));
	return XALM_OK;
}

// beyond the matrices: the visible cache rows, the recurrent state read and written; of a mixture only the chosen experts are read
long long active_bytes(SeqModel* sm, long long pos) {
	Du* m = static_cast<Du*>(sm);
	long long b = 0;
	const long long kelem = m->precision == XALM_PRECISION_F32 ? 4 : 2, welem = m->w_bf16 ? 2 : 4;
	for (const Layer& L : m->layers) {
		if (L.mixer == MIX_RETENTION) b += 2ll * L.H * L.d * L.dv * 4;
		else b += (pos + 1) * (L.R + L.r) * kelem;
		if (L.ff_kind == FF_MOE) b -= (long long) (L.E - L.top) * 3 * L.ff * m->width * welem;
	}
	return b;
}

bool state_buffer(SeqModel* sm, int layer, const float** src, size_t* count) {
	Du* m = static_cast<Du*>(sm);
	const Layer& L = m->layers[(size_t) layer];
	if (L.mixer != MIX_RETENTION) return false;
	*src = L.state;
	*count = (size_t) L.H * L.d * L.dv;
	return true;
}

void destroy(SeqModel* sm) {
	Du* m = static_cast<Du*>(sm);
	for (Layer& L : m->layers) {
		for (TcWeight* t : {&L.t_in, &L.t_o, &L.t_uq, &L.t_up, &L.t_down}) tc_weight_free(t);
		for (TcWeight& t : L.t_egu) tc_weight_free(&t);
		for (TcWeight& t : L.t_edown) tc_weight_free(&t);
	}
	if (m->h_off) cudaFreeHost(m->h_off);
	delete m;
}

const SeqHooks duletar_hooks = {parse_config, finalize, enqueue_pass, release, active_bytes, state_buffer, destroy};
extern const ModelFamily duletar_family;
int create(const char* json, int device, int max_tokens, int precision, xalm_cuda_model** out) {
	return seq_create<Du>(&duletar_family, &duletar_hooks, json, device, max_tokens, precision, out);
}
const ModelFamily duletar_family = seq_family_table("Duletar", create);
const FamilyRegistrar duletar_registrar(&duletar_family);

} // namespace
} // namespace xalm
