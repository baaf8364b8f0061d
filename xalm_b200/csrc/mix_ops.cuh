// mix_ops.cuh — sequence-mixing and layer-plumbing mechanisms for model families described by a config.json, each a kernel
// of its own with its constants as arguments so that another design can use it:
//
//   embed_streams_kernel   token rows -> S copies of the residual stream (hyper-connections; S = 1: the plain stream)
//   hc_norm_kernel         u = sum_s a[s] x_s, then RMS norm with a plain or one-plus weight (the read side of a hyper-connection
//                          fused with the pre-norm; S = 1, a = {1}: a plain pre-norm)
//   rows_gemm_kernel       out(T,N) = A(T,K) . W(N,K)^T in IEEE fp32 (weights bf16 or fp32), T > 4
//   rows_matvec_kernel     the same for T <= 4 (one-token steps): a warp per pair of output columns, 128-bit weight loads
//     both with the fused epilogues of RowsEpi: plain store; split store that sends the key / value columns of an input projection
//     straight into the ring cache; clamped GLU on interleaved gate|up columns; hyper-connection write (all streams updated from
//     the old ones, with the layer scale)
//   swa_attn_kernel        softmax attention over a sliding window with grouped K/V heads, tanh soft-capping, a logarithmic
//                          distance bias per head, a head-mixing matrix applied to the scores before the softmax and a sigmoid
//                          output gate; keys split over CTAs for one-token steps (swa_merge_kernel joins the parts)
//   hgrn2_kernel           gated linear recurrence S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T, o_t = S_t^T q_t with a lower-bounded
//                          forget gate, state in fp32 carried in device memory, per-head RMS norm of o fused
//   dual_norm_hc_kernel    y = 1/2 (rmsnorm(a) wa + rmsnorm(b) wb) -> layer scale -> hyper-connection write
//   group_norm_residual_kernel  x + grouped RMS norm of a sublayer's output (weighted sum of expert rows first), depth-weighted average
//   qkv_post_kernel        bias, rotary positions, weightless RMS norms of q / k / v heads, K/V cache write (kept first slots + ring)
//
// The kernels have internal linkage: every translation unit that includes this header (a model family, the op-level entry points
// of mix_ops.cu) gets its own copies.
//
// Numerics: everything here is fp32 (expf / tanhf / log1pf, no fast-math); 16-bit storage appears only as weight and K/V-cache
// element types.
#pragma once
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <algorithm>

#include "common.cuh"

namespace xalm {
namespace mix {

constexpr int MAX_STREAMS = 8;

// ---- element access ------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
// eight consecutive elements (16-byte aligned for bf16, 32-byte for fp32) -> fp32
__device__ __forceinline__ void ld8(const float* p, float* o) {
	const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
	o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float* o) {
	const uint4 r = *reinterpret_cast<const uint4*>(p);
	o[0] = __uint_as_float(r.x << 16); o[1] = __uint_as_float(r.x & 0xffff0000u);
	o[2] = __uint_as_float(r.y << 16); o[3] = __uint_as_float(r.y & 0xffff0000u);
	o[4] = __uint_as_float(r.z << 16); o[5] = __uint_as_float(r.z & 0xffff0000u);
	o[6] = __uint_as_float(r.w << 16); o[7] = __uint_as_float(r.w & 0xffff0000u);
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

// block-wide sum; every thread gets the result.  `red` holds 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
	v = warp_sum(v);
	const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
	__syncthreads();
	if (lane == 0) red[w] = v;
	__syncthreads();
	if (w == 0) {
		float t = lane < nw ? red[lane] : 0.f;
		t = warp_sum(t);
		if (lane == 0) red[32] = t;
	}
	__syncthreads();
	return red[32];
}

// what the kernels of one step read from device memory, so that a captured graph serves every position
struct SeqStep {
	int pos0; // position of the step's first token in its sequence
	int n;    // tokens in the step
	int prev; // the token before the step's first one, -1 at a sequence's start (designs whose embedding looks at token pairs)
};

// ---- embedding -> streams -------------------------------------------------------------------------------------------------
template <typename WT>
__global__ void embed_streams_kernel(const WT* __restrict__ table, const int* __restrict__ tokens, int width, int S, size_t stream_stride,
                                     float* __restrict__ xs, float scale = 1.f) {
	const int t = blockIdx.x;
	const WT* row = table + (size_t) tokens[t] * width;
	for (int c = threadIdx.x; c < width; c += blockDim.x) {
		const float v = ldf(row + c) * scale; // scale 1: the row as it is
		for (int s = 0; s < S; s++) xs[(size_t) s * stream_stride + (size_t) t * width + c] = v;
	}
}

// ---- embedding row + hashed token-pair row + grouped norm ------------------------------------------------------------------------------
// x[t] = gnorm(table[token] * scale + pair[(prev * mul_prev + token * mul_cur) mod buckets]) * w: the pair table's last row (number `buckets`)
// serves a sequence's first token, whose `prev` is the step's (SeqStep.prev < 0).  pair NULL: no pair rows; w NULL: no norm.  The norm is
// the grouped RMS norm of group_norm_residual_kernel.  One CTA per token; shared memory: width + groups floats.
struct EmbedPairArgs {
	const void* table; // (vocab, width) bf16 or fp32
	const void* pair;  // (buckets + 1, width) or NULL
	float scale;
	long long mul_prev, mul_cur;
	int buckets;
	const float* w;    // (width) or NULL
	int groups, width;
	float eps;
	const int* tokens;
	const SeqStep* step;
	float* x;          // (T, width)
};
template <typename WT>
__global__ void embed_pair_kernel(EmbedPairArgs a) {
	extern __shared__ float sm[];
	float* u = sm;
	float* rinv = sm + a.width;
	const int t = blockIdx.x, tid = threadIdx.x, nth = blockDim.x, lane = tid & 31, warp = tid >> 5, nw = nth >> 5;
	if (t >= a.step->n) return;
	const int W = a.width, tok = a.tokens[t], prev = t ? a.tokens[t - 1] : a.step->prev;
	const WT* row = reinterpret_cast<const WT*>(a.table) + (size_t) tok * W;
	const WT* prow = nullptr;
	if (a.pair) {
		const long long r = prev < 0 ? a.buckets : ((long long) prev * a.mul_prev + (long long) tok * a.mul_cur) % a.buckets;
		prow = reinterpret_cast<const WT*>(a.pair) + (size_t) r * W;
	}
	for (int c = tid; c < W; c += nth) {
		float v = ldf(row + c) * a.scale;
		if (prow) v += ldf(prow + c);
		u[c] = v;
	}
	__syncthreads();
	if (!a.w) {
		for (int c = tid; c < W; c += nth) a.x[(size_t) t * W + c] = u[c];
		return;
	}
	const int gs = W / a.groups;
	for (int g = warp; g < a.groups; g += nw) {
		float ss = 0.f;
		for (int c = lane; c < gs; c += 32) ss = fmaf(u[g * gs + c], u[g * gs + c], ss);
		ss = warp_sum(ss);
		if (lane == 0) rinv[g] = 1.f / sqrtf(ss / (float) gs + a.eps);
	}
	__syncthreads();
	for (int c = tid; c < W; c += nth) a.x[(size_t) t * W + c] = u[c] * rinv[c / gs] * a.w[c];
}

// ---- hyper-connection read + RMS norm -------------------------------------------------------------------------------------
// h[t] = rmsnorm(sum_s a[s] xs[s][t]) * (one_plus ? 1 + w : w).  a == nullptr: every coefficient is 1 (the final sum of streams).
// `sum_out` (optional) receives the un-normed combination (the residual stream as a reader outside the model sees it).
// SS: the most streams this instance takes (its loops are unrolled to SS: the code of a one-CTA launch should be short to fetch)
template <int SS>
__global__ void hc_norm_kernel(const float* __restrict__ xs, int S, size_t stream_stride, const float* __restrict__ a, const float* __restrict__ w,
                               int one_plus, float eps, int width, float* __restrict__ h, float* __restrict__ sum_out) {
	extern __shared__ float sm[];
	float* u = sm;            // width
	float* red = sm + width;  // 33
	const int t = blockIdx.x, tid = threadIdx.x, nth = blockDim.x;
	// Four columns per thread at a time, every load of the four issued before the first use: a one-token step runs one CTA of this
	// kernel, and its time is the number of dependent trips to memory.
	float av[SS];
#pragma unroll
	for (int s = 0; s < SS; s++) av[s] = (a && s < S) ? a[s] : 1.f;
	float ss = 0.f;
	for (int c0 = 0; c0 < width; c0 += 4 * nth) {
		float x[4][SS];
#pragma unroll
		for (int k = 0; k < 4; k++) {
			const int c = c0 + k * nth + tid;
#pragma unroll
			for (int s = 0; s < SS; s++) x[k][s] = (s < S && c < width) ? xs[(size_t) s * stream_stride + (size_t) t * width + c] : 0.f;
		}
#pragma unroll
		for (int k = 0; k < 4; k++) {
			const int c = c0 + k * nth + tid;
			float v = 0.f;
#pragma unroll
			for (int s = 0; s < SS; s++)
				if (s < S) v = a ? fmaf(av[s], x[k][s], v) : v + x[k][s];
			if (c < width) {
				u[c] = v;
				ss = fmaf(v, v, ss);
			}
		}
	}
	const float tot = block_sum(ss, red);
	const float r = 1.f / sqrtf(tot / (float) width + eps);
	for (int c0 = 0; c0 < width; c0 += 4 * nth) {
		float wv[4];
#pragma unroll
		for (int k = 0; k < 4; k++) {
			const int c = c0 + k * nth + tid;
			wv[k] = (h && c < width) ? w[c] : 0.f;
		}
#pragma unroll
		for (int k = 0; k < 4; k++) {
			const int c = c0 + k * nth + tid;
			if (c < width) {
				const float v = u[c];
				if (h) h[(size_t) t * width + c] = v * r * (one_plus ? 1.f + wv[k] : wv[k]);
				if (sum_out) sum_out[(size_t) t * width + c] = v;
			}
		}
	}
}

// ---- fused epilogues of the row products -------------------------------------------------------------------------------------
enum { EPI_STORE = 0, EPI_SPLIT_KV = 1, EPI_GLU = 2, EPI_HC = 3, EPI_ACT = 4 };
enum { GLU_CLAMPED = 0, GLU_SILU = 1, GLU_GELU_TANH = 2 };
enum { ACT_NONE = 0, ACT_RELU_SQUARED = 1, ACT_SIGMOID = 2, ACT_SILU = 3, ACT_GELU_TANH = 4, ACT_SIGMOID_POW = 5 };
struct RowsEpi {
	int kind = EPI_STORE;
	float* out = nullptr; // STORE / SPLIT_KV / ACT: (T, ldo); GLU: (T, ldo) with ldo = N / 2
	int ldo = 0;
	// STORE: v <- cap * tanh(v / cap) when cap > 0 (soft-capped logits); then v <- v * mul_act(mul[row * ldm + col]) when mul is set (an
	// output gate computed from the same input as the product's operand)
	float cap = 0.f;
	const float* mul = nullptr;
	int ldm = 0, mul_act = ACT_SIGMOID;
	// ACT: v <- act(v + bias[col]), no gate.  ACT_SIGMOID_POW: sigmoid(.)^act_pow, as exp(act_pow * log sigmoid(.)) (a decay in (0, 1) whose
	// logarithm stays exact where the sigmoid itself would leave the fp32 range)
	int act = ACT_NONE;
	const float* bias = nullptr;
	float act_pow = 1.f;
	// batched products (blockIdx.z = b): A advances by batch_a floats, W by batch_w elements, the output (and mul) by batch_o columns.
	// One launch then runs a product per head on that head's slice of the rows.
	int batch_a = 0, batch_o = 0;
	size_t batch_w = 0;
	// SPLIT_KV: columns [n_plain, n_plain + kdim) are the step's keys, the next vdim its values; they go to ring slot (pos0 + row) % ring
	int n_plain = 0, kdim = 0, vdim = 0, ring = 1, cache_f32 = 0;
	void* kc = nullptr;
	void* vc = nullptr;
	const SeqStep* step = nullptr;
	// SPLIT_KV, plain columns: [silu_off, silu_off + silu_n) -> z * sigmoid(z); [gate_off, gate_off + gate_n) -> a lower-bounded sigmoid gate
	// lo + (1 - lo) * sigmoid(z + bias) with lo = gate_lower[col - gate_off] (NULL: 0) and bias = gate_bias[col - gate_off] (NULL: 0)
	int silu_off = 0, silu_n = 0, gate_off = 0, gate_n = 0;
	const float* gate_bias = nullptr;
	const float* gate_lower = nullptr;
	// GLU: even column = gate, odd = up.  glu_act GLU_CLAMPED: y = min(g, limit) * sigmoid(alpha * .) * (clamp(u, +-limit) + 1);
	// GLU_SILU: y = g sigmoid(g) u;  GLU_GELU_TANH: y = 1/2 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) u
	float limit = 0.f, alpha = 1.702f;
	int glu_act = 0;
	// HC: xs[t'][row][col] = sum_s hmix[s * S + t'] xs[s][row][col] + hout[t'] * scale[col] * value   (hmix / hout NULL: identity / ones)
	float* xs = nullptr;
	int S = 1;
	size_t stream_stride = 0;
	const float* hmix = nullptr;
	const float* hout = nullptr;
	const float* scale = nullptr; // layer scale (NULL: none)
};

__device__ __forceinline__ float glu_clamped(float g, float u, float limit, float alpha) {
	g = fminf(g, limit);
	u = fminf(fmaxf(u, -limit), limit);
	return g * sigmoidf_(alpha * g) * (u + 1.f);
}

__device__ __forceinline__ float gelu_tanhf_(float z) { return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }
__device__ __forceinline__ float log_sigmoidf_(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float act_apply(int act, float v, float p = 1.f) {
	if (act == ACT_RELU_SQUARED) { v = fmaxf(v, 0.f); return v * v; }
	if (act == ACT_SIGMOID) return sigmoidf_(v);
	if (act == ACT_SILU) return v * sigmoidf_(v);
	if (act == ACT_GELU_TANH) return gelu_tanhf_(v);
	if (act == ACT_SIGMOID_POW) return expf(p * log_sigmoidf_(v));
	return v;
}
__device__ __forceinline__ float glu_apply(int act, float g, float u, float limit, float alpha) {
	if (act == GLU_SILU) return g * sigmoidf_(g) * u;
	if (act == GLU_GELU_TANH) return gelu_tanhf_(g) * u;
	return glu_clamped(g, u, limit, alpha);
}

__device__ __forceinline__ void hc_write(const RowsEpi& e, int row, int col, int width, float v) {
	const float y = e.scale ? e.scale[col] * v : v;
	float old[MAX_STREAMS];
	const size_t at = (size_t) row * width + col;
	for (int s = 0; s < e.S; s++) old[s] = e.xs[(size_t) s * e.stream_stride + at];
	for (int t = 0; t < e.S; t++) {
		float acc;
		if (e.hmix) {
			acc = 0.f;
			for (int s = 0; s < e.S; s++) acc = fmaf(e.hmix[s * e.S + t], old[s], acc);
		} else acc = old[t];
		e.xs[(size_t) t * e.stream_stride + at] = fmaf(e.hout ? e.hout[t] : 1.f, y, acc);
	}
}

// one value (for the pairwise GLU: called with the even column and both values)
__device__ __forceinline__ void epi_apply(const RowsEpi& e, int row, int col, int N, float v, float v_next) {
	switch (e.kind) {
		case EPI_STORE:
			if (e.cap > 0.f) v = e.cap * tanhf(v / e.cap);
			if (e.mul) v *= act_apply(e.mul_act, e.mul[(size_t) row * e.ldm + col]);
			e.out[(size_t) row * e.ldo + col] = v;
			break;
		case EPI_ACT: e.out[(size_t) row * e.ldo + col] = act_apply(e.act, e.bias ? v + e.bias[col] : v, e.act_pow); break;
		case EPI_SPLIT_KV: {
			if (col < e.n_plain) {
				if (col >= e.silu_off && col < e.silu_off + e.silu_n) v = v * sigmoidf_(v);
				else if (col >= e.gate_off && col < e.gate_off + e.gate_n) {
					const int c = col - e.gate_off;
					const float lo = e.gate_lower ? e.gate_lower[c] : 0.f;
					v = lo + (1.f - lo) * sigmoidf_(v + (e.gate_bias ? e.gate_bias[c] : 0.f));
				}
				e.out[(size_t) row * e.ldo + col] = v;
				break;
			}
			const int slot = (e.step->pos0 + row) % e.ring;
			const int ck = col - e.n_plain;
			if (ck < e.kdim) {
				if (e.cache_f32) ((float*) e.kc)[(size_t) slot * e.kdim + ck] = v;
				else ((__nv_bfloat16*) e.kc)[(size_t) slot * e.kdim + ck] = __float2bfloat16_rn(v);
			} else {
				const int cv = ck - e.kdim;
				if (e.cache_f32) ((float*) e.vc)[(size_t) slot * e.vdim + cv] = v;
				else ((__nv_bfloat16*) e.vc)[(size_t) slot * e.vdim + cv] = __float2bfloat16_rn(v);
			}
			break;
		}
		case EPI_GLU: e.out[(size_t) row * e.ldo + (col >> 1)] = glu_apply(e.glu_act, v, v_next, e.limit, e.alpha); break;
		case EPI_HC: hc_write(e, row, col, N, v); break;
	}
}

// ---- out(T,N) = A(T,K) . W(N,K)^T, fp32 FMA, 64x64x16 tiles, 4x4 per thread ---------------------------------------------------
template <typename WT>
__global__ void __launch_bounds__(256) rows_gemm_kernel(const float* __restrict__ A, int lda, const WT* __restrict__ W, int T, int N, int K, RowsEpi e) {
	constexpr int BM = 64, BN = 64, BK = 16;
	if (blockIdx.z) { // one product of a batch
		A += (size_t) blockIdx.z * e.batch_a;
		W += (size_t) blockIdx.z * e.batch_w;
		e.out += (size_t) blockIdx.z * e.batch_o;
		if (e.mul) e.mul += (size_t) blockIdx.z * e.batch_o;
	}
	__shared__ float As[BK][BM + 4];
	__shared__ float Ws[BK][BN + 4];
	const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
	const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
	float acc[4][4] = {};
	for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
		for (int i = 0; i < 4; i++) {
			const int idx = tid + i * 256; // 0..1023: r = idx / 16, k = idx % 16 (k fastest: coalesced along K)
			const int r = idx >> 4, k = idx & 15;
			const int gm = m0 + r, gn = n0 + r, gk = k0 + k;
			As[k][r] = (gm < T && gk < K) ? A[(size_t) gm * lda + gk] : 0.f;
			Ws[k][r] = (gn < N && gk < K) ? ldf(W + (size_t) gn * K + gk) : 0.f;
		}
		__syncthreads();
#pragma unroll
		for (int k = 0; k < BK; k++) {
			const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
			const float4 b = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
			const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
			for (int i = 0; i < 4; i++)
#pragma unroll
				for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
		}
		__syncthreads();
	}
#pragma unroll
	for (int i = 0; i < 4; i++) {
		const int row = m0 + ty * 4 + i;
		if (row >= T) continue;
		if (e.kind == EPI_GLU) {
#pragma unroll
			for (int j = 0; j < 4; j += 2) {
				const int col = n0 + tx * 4 + j;
				if (col + 1 < N) epi_apply(e, row, col, N, acc[i][j], acc[i][j + 1]);
			}
		} else {
#pragma unroll
			for (int j = 0; j < 4; j++) {
				const int col = n0 + tx * 4 + j;
				if (col < N) epi_apply(e, row, col, N, acc[i][j], 0.f);
			}
		}
	}
}

// ---- the epilogues alone, on a product that another kernel left in memory (the tensor-core GEMM stores plain fp32 rows) --------------
static __global__ void rows_epilogue_kernel(const float* __restrict__ src, int lds, int T, int N, RowsEpi e) {
	const int step = e.kind == EPI_GLU ? 2 : 1, per_row = (N + step - 1) / step;
	const size_t total = (size_t) T * per_row;
	for (size_t i = blockIdx.x * (size_t) blockDim.x + threadIdx.x; i < total; i += (size_t) gridDim.x * blockDim.x) {
		const int row = (int) (i / per_row), col = (int) (i % per_row) * step;
		const float* p = src + (size_t) row * lds + col;
		if (step == 2) {
			if (col + 1 < N) epi_apply(e, row, col, N, p[0], p[1]);
		} else epi_apply(e, row, col, N, p[0], 0.f);
	}
}

// ---- the same for T <= TB tokens: a warp per pair of output columns, or KS warps of the CTA per pair (each a slice of K, summed through
// shared memory) when there are too few columns to fill the machine ---------------------------------------------------------------
template <typename WT, int TB, int KS>
__global__ void __launch_bounds__(256) rows_matvec_kernel(const float* __restrict__ A, int lda, const WT* __restrict__ W, int T, int N, int K, RowsEpi e) {
	__shared__ float red[8][TB][2];
	if (blockIdx.z) { // one product of a batch
		A += (size_t) blockIdx.z * e.batch_a;
		W += (size_t) blockIdx.z * e.batch_w;
		e.out += (size_t) blockIdx.z * e.batch_o;
		if (e.mul) e.mul += (size_t) blockIdx.z * e.batch_o;
	}
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, ks = warp % KS;
	const int pair = blockIdx.x * (8 / KS) + warp / KS;
	const int c0 = pair * 2;
	const bool live = c0 < N, two = c0 + 1 < N;
	float acc0[TB] = {}, acc1[TB] = {};
	if (live) {
		const WT* w0 = W + (size_t) c0 * K;
		const WT* w1 = W + (size_t) (two ? c0 + 1 : c0) * K;
		const bool vec = (K % 8 == 0) && (lda % 4 == 0) && ((reinterpret_cast<uintptr_t>(W) & 31) == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0); // of this batch's slices
		if (vec) {
#pragma unroll 2
			for (int k = (ks * 32 + lane) * 8; k < K; k += 256 * KS) {
				float a0[8], a1[8];
				ld8(w0 + k, a0);
				ld8(w1 + k, a1);
#pragma unroll
				for (int t = 0; t < TB; t++) {
					if (t < T) {
						float x[8];
						ld8(A + (size_t) t * lda + k, x);
#pragma unroll
						for (int i = 0; i < 8; i++) {
							acc0[t] = fmaf(a0[i], x[i], acc0[t]);
							acc1[t] = fmaf(a1[i], x[i], acc1[t]);
						}
					}
				}
			}
		} else {
			for (int k = ks * 32 + lane; k < K; k += 32 * KS) {
				const float a0 = ldf(w0 + k), a1 = ldf(w1 + k);
#pragma unroll
				for (int t = 0; t < TB; t++)
					if (t < T) {
						const float x = A[(size_t) t * lda + k];
						acc0[t] = fmaf(a0, x, acc0[t]);
						acc1[t] = fmaf(a1, x, acc1[t]);
					}
			}
		}
#pragma unroll
		for (int t = 0; t < TB; t++) {
			acc0[t] = warp_sum(acc0[t]);
			acc1[t] = warp_sum(acc1[t]);
		}
	}
	if (KS > 1) {
		if (lane == 0)
#pragma unroll
			for (int t = 0; t < TB; t++) { red[warp][t][0] = acc0[t]; red[warp][t][1] = acc1[t]; }
		__syncthreads();
		if (ks == 0 && lane == 0)
#pragma unroll
			for (int t = 0; t < TB; t++)
				for (int j = 1; j < KS; j++) { acc0[t] += red[warp + j][t][0]; acc1[t] += red[warp + j][t][1]; }
	}
	if (live && ks == 0 && lane == 0) {
#pragma unroll
		for (int t = 0; t < TB; t++) {
			if (t >= T) break;
			if (e.kind == EPI_GLU) {
				if (two) epi_apply(e, t, c0, N, acc0[t], acc1[t]);
			} else {
				epi_apply(e, t, c0, N, acc0[t], 0.f);
				if (two) epi_apply(e, t, c0 + 1, N, acc1[t], 0.f);
			}
		}
	}
}

// ---- sliding-window softmax attention with score mixing across heads -------------------------------------------------------------
struct SwaArgs {
	const float* q;    // (T, ldq): head h at columns q_off + h * d
	const float* gate; // (T, ldg): pre-sigmoid gate of the concatenated heads at columns g_off + ...; NULL: no gate
	int ldq, q_off, ldg, g_off;
	const void* kc;    // ring (ring, G * d)
	const void* vc;    // ring (ring, G * dv)
	int ldk, ldv;      // elements between the rows of two slots; 0: G * d and G * dv.  A cache whose rows hold more than the keys (values that
	                   // are a slice of the key row: vc points into kc with ldv = ldk) is read in place
	int ring;
	int H, G, d, dv;
	int window;        // position i sees j with 0 <= i - j < window
	int keep_first;    // ... and every j < keep_first (j <= i) however far back: the sequence's first positions stay visible at their true
	                   // places.  They live in slots [0, keep_first) of the cache, the others in the `ring` slots behind (0: a plain ring)
	float scale;
	float softcap;     // 0: none
	const float* r1;   // distance bias r1[h] * log1p(r2[h] * (i - j)) taken off the score; NULL: none
	const float* r2;
	const float* talk; // (H, H) score_h <- sum_g talk[h, g] score_g; NULL: none
	const float* sink; // (H) the softmax's denominator also holds exp(sink[h]): a key of no position and no value that is not scaled; NULL: none
	float out_scale;   // multiplies the result (0: 1)
	const SeqStep* step;
	float* out;        // (T, ldo): head h at columns h * dv
	int ldo;           // 0: H * dv.  The launcher runs the heads of a single-group attention in several launches when all of them do not fit one
	                   // CTA's shared memory: each launch sees its share of the heads as H and the full row as ldo
	int n_splits;      // > 1: partial results to part_*; swa_merge_kernel finishes.  0: the launcher chooses (part_cap bounds it)
	int part_cap;      // (row, split) pairs part_o / part_ml have room for (only read when n_splits == 0)
	int tq;            // queries per CTA of the tiled kernel (set by the launcher)
	int stage_off;     // one-query kernel: > 0: the key block's K and V rows are copied (cp.async, 16 bytes) to shared memory at this float offset
	                   // before they are used, so that a CTA's time is a few trips to memory (set by the launcher)
	unsigned* tickets; // one zeroed counter per query tile, or NULL.  With it the tiled kernel's last-arriving key split joins the parts itself
	                   // (and resets the counter); without it swa_merge_kernel follows
	float* part_o;     // (T, n_splits, H * dv)
	float* part_ml;    // (T, n_splits, H, 2)
};

constexpr int SWA_KB = 32; // keys per block

// The keys a CTA's queries [i_lo, i_hi] can see, as one run of "virtual" indices: first the kept positions that have left the window of
// i_lo, then the positions from the window's start on.  pos(): the position in the sequence; slot(): where the cache keeps it.
struct SwaKeys {
	int j_first, ks, keep, ring;
	__device__ __forceinline__ int pos(int v) const { return v < ks ? v : j_first + (v - ks); }
	__device__ __forceinline__ int slot(int v) const {
		const int j = pos(v);
		return j < keep ? j : keep + (j - keep) % ring;
	}
};
__device__ __forceinline__ SwaKeys swa_keys(int window, int keep_first, int ring, int i_lo) {
	SwaKeys k;
	k.j_first = window < 0x7fffffff ? max(0, i_lo - window + 1) : 0;
	k.ks = min(keep_first, k.j_first);
	k.keep = keep_first;
	k.ring = ring;
	return k;
}

// o = num / (den + exp(sink - m)), num and den being sums of exp(score - m); written so that a sink far above every score cannot overflow
__device__ __forceinline__ float swa_finish(const SwaArgs& a, int h, float num, float den, float m) {
	if (a.sink) {
		const float sk = a.sink[h];
		if (sk > m) {
			const float c = expf(m - sk);
			num *= c;
			den = fmaf(den, c, 1.f);
		} else den += expf(sk - m);
	}
	const float o = num / den;
	return a.out_scale != 0.f ? o * a.out_scale : o;
}

// joins the key splits of rows [t_first, t_first + rows): out = (sum_s e^{m_s - m} O_s) / (sum_s e^{m_s - m} l_s), then the gate
__device__ __forceinline__ void swa_merge_one(const SwaArgs& a, int t, int hc) {
	const int H = a.H, dv = a.dv, ns = a.n_splits, h = hc / dv;
	const float* pml0 = a.part_ml + (size_t) t * ns * (H * 2) + 2 * h;
	const float* po0 = a.part_o + (size_t) t * ns * (H * dv) + hc;
	float m = -INFINITY, num = 0.f, den = 0.f;
	for (int s0 = 0; s0 < ns; s0 += 8) { // eight splits' loads in flight, then one rescale for the eight
		float ms[8], ls[8], os[8];
#pragma unroll
		for (int u = 0; u < 8; u++) {
			const bool in = s0 + u < ns;
			ms[u] = in ? __ldcg(pml0 + (size_t) (s0 + u) * (H * 2)) : -INFINITY;
			ls[u] = in ? __ldcg(pml0 + (size_t) (s0 + u) * (H * 2) + 1) : 0.f;
			os[u] = in ? __ldcg(po0 + (size_t) (s0 + u) * (H * dv)) : 0.f;
		}
		float mb = m;
#pragma unroll
		for (int u = 0; u < 8; u++) mb = fmaxf(mb, ms[u]);
		if (mb == -INFINITY) continue;
		const float keep = m == -INFINITY ? 0.f : expf(m - mb);
		num *= keep;
		den *= keep;
		m = mb;
#pragma unroll
		for (int u = 0; u < 8; u++)
			if (ms[u] != -INFINITY) {
				const float w = expf(ms[u] - m);
				num = fmaf(w, os[u], num);
				den = fmaf(w, ls[u], den);
			}
	}
	float o = swa_finish(a, h, num, den, m);
	if (a.gate) o *= sigmoidf_(a.gate[(size_t) t * a.ldg + a.g_off + hc]);
	a.out[(size_t) t * (a.ldo ? a.ldo : H * dv) + hc] = o;
}
__device__ __forceinline__ void swa_merge_rows(const SwaArgs& a, int t_first, int rows, int tid, int nth) {
	const int hdv = a.H * a.dv;
	for (int x = tid; x < rows * hdv; x += nth) swa_merge_one(a, t_first + x / hdv, x % hdv);
}
// grid (rows, ceil(H dv / 128)), 128 threads: a thread per output value, so that a one-token step's join is spread over many SMs
static __global__ void swa_merge_kernel(SwaArgs a) {
	const int hc = blockIdx.y * blockDim.x + threadIdx.x;
	if (hc < a.H * a.dv) swa_merge_one(a, blockIdx.x, hc);
}

// With key splits and a ticket counter per query tile: the split that arrives last joins the parts of the tile's rows and leaves the
// counter at zero for the next launch.  Every thread of the CTA calls it after writing its parts.
__device__ __forceinline__ void swa_join_last(const SwaArgs& a, int tile, int t_first, int rows, int tid, int nth) {
	__shared__ int last;
	__threadfence();
	__syncthreads();
	if (tid == 0) {
		const unsigned got = atomicAdd(a.tickets + tile, 1u);
		last = got == (unsigned) a.n_splits - 1u;
		if (last) a.tickets[tile] = 0u;
	}
	__syncthreads();
	if (last) {
		__threadfence();
		swa_merge_rows(a, t_first, rows, tid, nth);
	}
}


template <typename CT>
__global__ void __launch_bounds__(256) swa_attn_kernel(SwaArgs a) {
	extern __shared__ float sm[];
	const int H = a.H, G = a.G, d = a.d, dv = a.dv, rep = H / G;
	float* qs = sm;                  // H * d
	float* sc = qs + H * d;          // H * KB raw scores
	float* pr = sc + H * SWA_KB;     // H * KB mixed scores, then probabilities
	float* tk = pr + H * SWA_KB;     // H * H
	float* mrun = tk + H * H;        // H
	float* lrun = mrun + H;          // H
	float* alpha = lrun + H;         // H
	float* O = alpha + H;            // H * dv
	const CT* kc = reinterpret_cast<const CT*>(a.kc);
	const CT* vc = reinterpret_cast<const CT*>(a.vc);
	const int t = blockIdx.x, sp = blockIdx.y, tid = threadIdx.x, nth = blockDim.x, lane = tid & 31, warp = tid >> 5, nw = nth >> 5;
	const int ldk = a.ldk ? a.ldk : G * d, ldv = a.ldv ? a.ldv : G * dv;
	const bool vec8 = ((d | ldk) & 7) == 0 && (reinterpret_cast<uintptr_t>(a.kc) & 31) == 0;
	if (t >= a.step->n) return;
	const int i = a.step->pos0 + t;
	const SwaKeys km = swa_keys(a.window, a.keep_first, a.ring, i);
	const int nk = km.ks + i - km.j_first + 1; // every one of them is visible to this query
	int per = (nk + a.n_splits - 1) / a.n_splits;
	per = (per + SWA_KB - 1) / SWA_KB * SWA_KB;
	const int jb = sp * per, je = min(nk, jb + per); // virtual key indices
	// staged rows: Ks[jj][G d], Vs[jj][G dv] in the cache's element type
	const bool staged = a.stage_off > 0;
	// one key/value head whose values are the first dv entries of the key rows (a latent cache): the staged key rows serve as values too
	const bool v_in_k = a.vc == a.kc && ldv == ldk && G == 1 && dv <= d;
	const int vs_ld = v_in_k ? G * d : G * dv;
	CT* Ks = reinterpret_cast<CT*>(sm + a.stage_off);
	CT* Vs = v_in_k ? Ks : Ks + (size_t) SWA_KB * G * d;
	auto stage = [&](int j0, int nb) {
		constexpr int EPC = 16 / (int) sizeof(CT); // elements per 16-byte copy
		const int kch = G * d / EPC, vch = G * dv / EPC;
		for (int x = tid; x < nb * kch; x += nth) {
			const int jj = x / kch, c = (x % kch) * EPC;
			const unsigned dst = (unsigned) __cvta_generic_to_shared(Ks + (size_t) jj * (G * d) + c);
			asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(kc + (size_t) km.slot(j0 + jj) * ldk + c) : "memory");
		}
		for (int x = tid; x < (v_in_k ? 0 : nb * vch); x += nth) {
			const int jj = x / vch, c = (x % vch) * EPC;
			const unsigned dst = (unsigned) __cvta_generic_to_shared(Vs + (size_t) jj * (G * dv) + c);
			asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(vc + (size_t) km.slot(j0 + jj) * ldv + c) : "memory");
		}
		asm volatile("cp.async.commit_group;" ::: "memory");
	};
	if (staged && jb < je) stage(jb, min(SWA_KB, je - jb)); // in flight while the query and the constants are read

	if (((a.ldq | a.q_off | (H * d)) & 3) == 0) {
#pragma unroll 4
		for (int x = tid * 4; x < H * d; x += nth * 4) *reinterpret_cast<float4*>(qs + x) = *reinterpret_cast<const float4*>(a.q + (size_t) t * a.ldq + a.q_off + x);
	} else
		for (int x = tid; x < H * d; x += nth) qs[x] = a.q[(size_t) t * a.ldq + a.q_off + x];
	for (int x = tid; x < H * H; x += nth) tk[x] = a.talk ? a.talk[x] : (x / H == x % H ? 1.f : 0.f);
	for (int x = tid; x < H; x += nth) { mrun[x] = -INFINITY; lrun[x] = 0.f; }
	for (int x = tid; x < H * dv; x += nth) O[x] = 0.f;
	__syncthreads();

	for (int j0 = jb; j0 < je; j0 += SWA_KB) {
		const int nb = min(SWA_KB, je - j0);
		if (staged) {
			if (j0 != jb) {
				__syncthreads(); // the last reader of the staged rows is done
				stage(j0, nb);
			}
			asm volatile("cp.async.wait_all;" ::: "memory");
			__syncthreads();
		}
		// raw scores: a warp takes keys warp, warp + 8, ... of the block (four with 256 threads), its lanes along the channels, eight
		// each; the loads of all four keys are issued before the first product, and up to four heads of the group share them.
		// Then scale, soft cap, distance bias.
		for (int g = 0; g < G; g++)
			for (int hr = 0; hr < rep; hr += 4) {
				const float* qh = qs + (size_t) (g * rep + hr) * d;
				const int nh = min(4, rep - hr);
				float acc[4][4] = {}; // [key][head]
				for (int c = lane * 8; c < d; c += 256) {
					float kk[4][8];
#pragma unroll
					for (int kq = 0; kq < 4; kq++) {
						const int jj = warp + kq * 8;
						const CT* kr = (staged ? Ks + (size_t) jj * (G * d) : kc + (size_t) km.slot(j0 + min(jj, nb - 1)) * ldk) + g * d + c;
						if (jj < nb && vec8) ld8(kr, kk[kq]);
						else
#pragma unroll
							for (int e8 = 0; e8 < 8; e8++) kk[kq][e8] = (jj < nb && c + e8 < d) ? ldf(kr + e8) : 0.f;
					}
#pragma unroll
					for (int u = 0; u < 4; u++)
						if (u < nh) {
							float qv[8];
							if (vec8) {
								const float4 q0 = *reinterpret_cast<const float4*>(qh + u * d + c), q1 = *reinterpret_cast<const float4*>(qh + u * d + c + 4);
								qv[0] = q0.x; qv[1] = q0.y; qv[2] = q0.z; qv[3] = q0.w; qv[4] = q1.x; qv[5] = q1.y; qv[6] = q1.z; qv[7] = q1.w;
							} else
#pragma unroll
								for (int e8 = 0; e8 < 8; e8++) qv[e8] = c + e8 < d ? qh[u * d + c + e8] : 0.f;
#pragma unroll
							for (int kq = 0; kq < 4; kq++)
#pragma unroll
								for (int e8 = 0; e8 < 8; e8++) acc[kq][u] = fmaf(qv[e8], kk[kq][e8], acc[kq][u]);
						}
				}
				float mine = 0.f; // lane kq * 4 + u keeps the sum of (key kq, head u)
#pragma unroll
				for (int kq = 0; kq < 4; kq++)
#pragma unroll
					for (int u = 0; u < 4; u++) {
						const float tot = warp_sum(acc[kq][u]);
						if (lane == kq * 4 + u) mine = tot;
					}
				if (lane < 16) {
					const int kq = lane >> 2, u = lane & 3, jj = warp + kq * 8, j = km.pos(j0 + jj);
					if (u < nh) {
						const int h = g * rep + hr + u;
						float sv = 0.f;
						if (jj < nb) {
							sv = mine * a.scale;
							if (a.softcap > 0.f) sv = a.softcap * tanhf(sv / a.softcap);
							if (a.r1) sv -= a.r1[h] * log1pf(a.r2[h] * (float) (i - j));
						}
						sc[h * SWA_KB + jj] = sv;
					}
				}
			}
		__syncthreads();
		// mix the heads' scores
		for (int x = tid; x < H * SWA_KB; x += nth) {
			const int h = x / SWA_KB, jj = x % SWA_KB;
			float s = -INFINITY;
			if (jj < nb) {
				if (a.talk) {
					s = 0.f;
					for (int g = 0; g < H; g++) s = fmaf(tk[h * H + g], sc[g * SWA_KB + jj], s);
				} else s = sc[x];
			}
			pr[x] = s;
		}
		__syncthreads();
		// online softmax, a warp per head
		for (int h = warp; h < H; h += nw) {
			const float s = pr[h * SWA_KB + lane]; // SWA_KB == 32
			const float bm = warp_max(s);
			const float m_old = mrun[h], m_new = fmaxf(m_old, bm);
			const float p = (lane < nb) ? expf(s - m_new) : 0.f;
			const float ps = warp_sum(p);
			pr[h * SWA_KB + lane] = p;
			if (lane == 0) {
				const float al = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
				alpha[h] = al;
				mrun[h] = m_new;
				lrun[h] = lrun[h] * al + ps;
			}
		}
		__syncthreads();
		// O <- alpha O + P V: a thread per value column of a kv group, up to four heads of the group per read of V
		for (int x = tid; x < G * dv; x += nth) {
			const int g = x / dv, c = x % dv;
			const CT* vcol = (staged ? Vs : vc) + g * dv + c;
			for (int hr = 0; hr < rep; hr += 4) {
				const int h0 = g * rep + hr, nh = min(4, rep - hr);
				float acc[4];
#pragma unroll
				for (int u = 0; u < 4; u++) acc[u] = u < nh ? O[(size_t) (h0 + u) * dv + c] * alpha[h0 + u] : 0.f;
				for (int jb8 = 0; jb8 < nb; jb8 += 8) { // eight loads in flight
					float v[8];
#pragma unroll
					for (int e8 = 0; e8 < 8; e8++) v[e8] = jb8 + e8 < nb ? ldf(vcol + (staged ? (size_t) (jb8 + e8) * vs_ld : (size_t) km.slot(j0 + jb8 + e8) * ldv)) : 0.f;
#pragma unroll
					for (int e8 = 0; e8 < 8; e8++)
#pragma unroll
						for (int u = 0; u < 4; u++)
							if (u < nh) acc[u] = fmaf(pr[(h0 + u) * SWA_KB + jb8 + e8], v[e8], acc[u]);
				}
#pragma unroll
				for (int u = 0; u < 4; u++)
					if (u < nh) O[(size_t) (h0 + u) * dv + c] = acc[u];
			}
		}
		__syncthreads();
	}
	if (a.n_splits == 1) {
		for (int x = tid; x < H * dv; x += nth) {
			float o = swa_finish(a, x / dv, O[x], lrun[x / dv], mrun[x / dv]);
			if (a.gate) o *= sigmoidf_(a.gate[(size_t) t * a.ldg + a.g_off + x]);
			a.out[(size_t) t * (a.ldo ? a.ldo : H * dv) + x] = o;
		}
	} else {
		float* po = a.part_o + ((size_t) t * a.n_splits + sp) * (H * dv);
		float* pml = a.part_ml + ((size_t) t * a.n_splits + sp) * (H * 2);
		for (int x = tid; x < H * dv; x += nth) po[x] = O[x];
		for (int x = tid; x < H; x += nth) { pml[2 * x] = mrun[x]; pml[2 * x + 1] = lrun[x]; }
	}
}

// float offset of the staged rows behind the kernel's own arrays (16-byte aligned), and the bytes they take
inline size_t swa_stage_off(int H, int d, int dv) { return ((size_t) H * d + 2 * (size_t) H * SWA_KB + (size_t) H * H + 3 * (size_t) H + (size_t) H * dv + 3) & ~(size_t) 3; }
inline size_t swa_stage_bytes(int G, int d, int dv, bool cache_f32, bool v_in_k = false) { return (size_t) SWA_KB * G * (d + (v_in_k ? 0 : dv)) * (cache_f32 ? 4 : 2); }
inline size_t swa_smem_bytes(int H, int d, int dv) { return sizeof(float) * ((size_t) H * d + 2 * (size_t) H * SWA_KB + (size_t) H * H + 3 * (size_t) H + (size_t) H * dv); }


// ---- the same attention, tiled: a CTA takes `tq` consecutive queries with ALL their heads (the score mixing needs every head's score
// of a query-key pair) and walks the keys SWA_KB at a time ------------------------------------------------------------------------
// Rows of the tile are (kv group g, head in group, query): row = g * Rg + hr * tq + q with Rg = rep * tq rounded up to 4, so that the
// rows of one group are contiguous and share that group's K and V tile.  Per key block:
//   for every group: K tile -> shared memory; raw scores = 4x4 register tiles of Q . K^T (both row-major, float4 along the channel;
//                    a thread's 4 keys are 8 apart, which keeps the 16-byte loads of a quarter-warp on distinct banks);
//                    scale, soft cap, distance bias -> Sc[key][row]
//   mix heads (4 output heads per thread) and mask -> Pr[key][row];  online softmax, a warp per row
//   for every group: V tile -> shared memory; O[row][:] = alpha O + P^T . V in 4x4 register tiles (float4 along rows and columns)
// Keys can be split over blockIdx.y for short steps (swa_merge_kernel joins).  Everything is fp32; the cache element type only sets
// how K and V are loaded.
struct SwaTile {
	int tq, Rg, R, dp, ldq, dvp, Hp;
};
__host__ __device__ inline SwaTile swa_tile_dims(int H, int G, int d, int dv, int tq) {
	SwaTile t;
	t.tq = tq;
	t.Rg = ((H / G) * tq + 3) & ~3;
	t.R = G * t.Rg;
	t.dp = (d + 3) & ~3;
	t.ldq = t.dp + 4;
	t.dvp = (dv + 3) & ~3;
	t.Hp = (H + 3) & ~3;
	return t;
}
__host__ __device__ inline size_t swa_tile_smem_floats(int H, int G, int d, int dv, int tq) {
	const SwaTile t = swa_tile_dims(H, G, d, dv, tq);
	const size_t kv = (size_t) SWA_KB * (t.ldq > t.dvp ? t.ldq : t.dvp);
	return (size_t) t.R * t.ldq + kv + 2 * (size_t) SWA_KB * t.R + (size_t) t.R * t.dvp + (size_t) H * t.Hp + 3 * (size_t) t.R;
}

// rows j0 .. j0 + SWA_KB of one kv group's slice of the ring (w elements at column col0 of rows of row_elems) -> dst[jj * ldd + c] in fp32,
// zero beyond nbk rows and beyond w columns (up to wp).  16-byte loads, two in flight per thread, when the slice allows.
template <typename CT>
__device__ __forceinline__ void swa_load_tile(float* dst, int ldd, const CT* base, int row_elems, int col0, int w, int wp, int j0, int nbk, const SwaKeys& km,
                                              int tid, int nth) {
	if (((w | row_elems | col0) & 7) == 0 && (reinterpret_cast<uintptr_t>(base) & 31) == 0) {
		const int cpr = w >> 3, total = SWA_KB * cpr;
		for (int x0 = tid; x0 < total; x0 += 2 * nth) {
			float v[2][8];
#pragma unroll
			for (int u = 0; u < 2; u++) {
				const int x = x0 + u * nth, jj = x / cpr, c = (x % cpr) << 3;
				if (x < total && jj < nbk) ld8(base + (size_t) km.slot(j0 + jj) * row_elems + col0 + c, v[u]);
				else
#pragma unroll
					for (int i = 0; i < 8; i++) v[u][i] = 0.f;
			}
#pragma unroll
			for (int u = 0; u < 2; u++) {
				const int x = x0 + u * nth, jj = x / cpr, c = (x % cpr) << 3;
				if (x < total) {
					*reinterpret_cast<float4*>(dst + jj * ldd + c) = make_float4(v[u][0], v[u][1], v[u][2], v[u][3]);
					*reinterpret_cast<float4*>(dst + jj * ldd + c + 4) = make_float4(v[u][4], v[u][5], v[u][6], v[u][7]);
				}
			}
		}
	} else {
		for (int x = tid; x < SWA_KB * wp; x += nth) {
			const int jj = x / wp, k = x % wp;
			dst[jj * ldd + k] = (jj < nbk && k < w) ? ldf(base + (size_t) km.slot(j0 + jj) * row_elems + col0 + k) : 0.f;
		}
	}
}

// raw scores of one kv group's rows against the staged K tile: RT x KT register tiles (RT rows, KT keys 32 / KT apart), so that a
// tile with few rows per group still has work for every thread; then scale, soft cap, distance bias -> Sc[key][row]
template <int KT, int RT>
__device__ __forceinline__ void swa_qk_tiles(const SwaArgs& a, const float* Qs, const float* KV, float* Sc, int g, int Rg, int R, int ldq, int ldkv, int dp,
                                             int TQ, int rep, int nq, int nbk, int i_lo, int j0, const SwaKeys& km, int tid, int nth) {
	constexpr int NTK = SWA_KB / KT;
	for (int tile = tid; tile < (Rg / RT) * NTK; tile += nth) {
		const int mt = tile / NTK, nt = tile % NTK;
		const float* qp = Qs + (size_t) (g * Rg + RT * mt) * ldq;
		const float* kp = KV + nt * ldkv;
		float acc[RT][KT] = {};
		for (int k = 0; k < dp; k += 4) {
			float4 qv[RT], kv[KT];
#pragma unroll
			for (int i = 0; i < RT; i++) qv[i] = *reinterpret_cast<const float4*>(qp + i * ldq + k);
#pragma unroll
			for (int u = 0; u < KT; u++) kv[u] = *reinterpret_cast<const float4*>(kp + u * NTK * ldkv + k);
#pragma unroll
			for (int i = 0; i < RT; i++)
#pragma unroll
				for (int u = 0; u < KT; u++) {
					acc[i][u] = fmaf(qv[i].x, kv[u].x, acc[i][u]);
					acc[i][u] = fmaf(qv[i].y, kv[u].y, acc[i][u]);
					acc[i][u] = fmaf(qv[i].z, kv[u].z, acc[i][u]);
					acc[i][u] = fmaf(qv[i].w, kv[u].w, acc[i][u]);
				}
		}
#pragma unroll
		for (int u = 0; u < KT; u++) {
			const int jj = nt + NTK * u, j = km.pos(j0 + jj);
			float o4[RT];
#pragma unroll
			for (int i = 0; i < RT; i++) {
				const int rr = RT * mt + i, hr = rr / TQ, q = rr % TQ;
				float s = 0.f;
				if (hr < rep && q < nq && jj < nbk) {
					const int h = g * rep + hr;
					s = acc[i][u] * a.scale;
					if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
					if (a.r1) s -= a.r1[h] * log1pf(a.r2[h] * (float) max(i_lo + q - j, 0));
				}
				o4[i] = s;
			}
			float* sp = Sc + (size_t) jj * R + g * Rg + RT * mt;
			if (RT == 4) *reinterpret_cast<float4*>(sp) = make_float4(o4[0], o4[1], o4[RT - 2], o4[RT - 1]);
			else *reinterpret_cast<float2*>(sp) = make_float2(o4[0], o4[1]);
		}
	}
}

// O[row][:] <- alpha[row] O[row][:] + sum_key P[key][row] V[key][:] for one kv group's rows: 4 x CW register tiles (CW = 4 value columns, or 2
// when that leaves threads without a tile)
template <int CW>
__device__ __forceinline__ void swa_pv_tiles(const float* Pr, const float* KV, float* O, const float* alpha, int g, int Rg, int R, int ldkv, int dvp, int tid, int nth) {
	const int NTv = dvp / CW;
	for (int tile = tid; tile < (Rg >> 2) * NTv; tile += nth) {
		const int mt = tile / NTv, nt = tile % NTv, rb = g * Rg + 4 * mt;
		float acc[4][CW] = {};
#pragma unroll 8
		for (int jj = 0; jj < SWA_KB; jj++) {
			const float4 pv = *reinterpret_cast<const float4*>(Pr + (size_t) jj * R + rb);
			const float pa[4] = {pv.x, pv.y, pv.z, pv.w};
			float va[CW];
			if (CW == 4) {
				const float4 vv = *reinterpret_cast<const float4*>(KV + jj * ldkv + 4 * nt);
				va[0] = vv.x; va[1] = vv.y; va[CW - 2] = vv.z; va[CW - 1] = vv.w;
			} else {
				const float2 vv = *reinterpret_cast<const float2*>(KV + jj * ldkv + 2 * nt);
				va[0] = vv.x; va[1] = vv.y;
			}
#pragma unroll
			for (int i = 0; i < 4; i++)
#pragma unroll
				for (int u = 0; u < CW; u++) acc[i][u] = fmaf(pa[i], va[u], acc[i][u]);
		}
#pragma unroll
		for (int i = 0; i < 4; i++) {
			float* op = O + (size_t) (rb + i) * dvp + CW * nt;
			const float al = alpha[rb + i];
#pragma unroll
			for (int u = 0; u < CW; u++) op[u] = fmaf(al, op[u], acc[i][u]);
		}
	}
}

template <typename CT>
__global__ void __launch_bounds__(256) swa_tile_kernel(SwaArgs a) {
	extern __shared__ __align__(16) float sm[];
	const int H = a.H, G = a.G, d = a.d, dv = a.dv, rep = H / G, TQ = a.tq;
	const SwaTile z = swa_tile_dims(H, G, d, dv, TQ);
	const int Rg = z.Rg, R = z.R, dp = z.dp, ldq = z.ldq, dvp = z.dvp, Hp = z.Hp;
	const int ldkv = ldq > dvp ? ldq : dvp;
	const int kt = (Rg >> 2) * 8 >= (int) blockDim.x ? 4 : (Rg >> 2) * 16 >= (int) blockDim.x ? 2 : 1; // keys per thread of the score tiles
	float* Qs = sm;                          // R * ldq
	float* KV = Qs + (size_t) R * ldq;       // SWA_KB * ldkv: one group's K tile, later its V tile
	float* Sc = KV + (size_t) SWA_KB * ldkv; // SWA_KB * R raw scores
	float* Pr = Sc + (size_t) SWA_KB * R;    // SWA_KB * R mixed scores, then probabilities
	float* O = Pr + (size_t) SWA_KB * R;     // R * dvp
	float* tkT = O + (size_t) R * dvp;       // H * Hp: tkT[g * Hp + h] = talk[h, g]
	float* mrun = tkT + (size_t) H * Hp;     // R
	float* lrun = mrun + R;                  // R
	float* alpha = lrun + R;                 // R
	const CT* kc = reinterpret_cast<const CT*>(a.kc);
	const CT* vc = reinterpret_cast<const CT*>(a.vc);
	const int tid = threadIdx.x, nth = blockDim.x, lane = tid & 31, warp = tid >> 5, nw = nth >> 5;
	const int n = a.step->n, pos0 = a.step->pos0;
	const int t0 = blockIdx.x * TQ, sp = blockIdx.y;
	const int nq = min(TQ, n - t0);          // queries of this tile (<= 0: nothing to do)
	if (nq <= 0) return;
	const int i_lo = pos0 + t0, i_hi = i_lo + nq - 1;
	const SwaKeys km = swa_keys(a.window, a.keep_first, a.ring, i_lo);
	const int nk = km.ks + i_hi - km.j_first + 1;
	int per = (nk + a.n_splits - 1) / a.n_splits;
	per = (per + SWA_KB - 1) / SWA_KB * SWA_KB;
	const int jb = sp * per, je = min(nk, jb + per); // virtual key indices

	// ---- Q tile (zero rows where the tile has no head or no query), constants ----
	for (int x = tid; x < R * (dp >> 2); x += nth) {
		const int row = x / (dp >> 2), k4 = (x % (dp >> 2)) << 2;
		const int g = row / Rg, rr = row % Rg, hr = rr / TQ, q = rr % TQ;
		float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
		if (hr < rep && q < nq) {
			const float* src = a.q + (size_t) (t0 + q) * a.ldq + a.q_off + (g * rep + hr) * d + k4;
			v.x = src[0];
			if (k4 + 1 < d) v.y = src[1];
			if (k4 + 2 < d) v.z = src[2];
			if (k4 + 3 < d) v.w = src[3];
		}
		*reinterpret_cast<float4*>(Qs + (size_t) row * ldq + k4) = v;
	}
	for (int x = tid; x < H * Hp; x += nth) {
		const int g = x / Hp, h = x % Hp;
		tkT[x] = h < H ? (a.talk ? a.talk[h * H + g] : (h == g ? 1.f : 0.f)) : 0.f;
	}
	for (int x = tid; x < R; x += nth) { mrun[x] = -INFINITY; lrun[x] = 0.f; alpha[x] = 0.f; }
	for (int x = tid; x < R * dvp; x += nth) O[x] = 0.f;

	for (int j0 = jb; j0 < je; j0 += SWA_KB) {
		const int nbk = min(SWA_KB, je - j0);
		// ---- raw scores, one kv group at a time ----
		for (int g = 0; g < G; g++) {
			__syncthreads(); // the last reader of KV (and, on the first pass, the set-up above) is done
			swa_load_tile(KV, ldkv, kc, a.ldk ? a.ldk : G * d, g * d, d, dp, j0, nbk, km, tid, nth);
			__syncthreads();
			if (kt == 4) swa_qk_tiles<4, 4>(a, Qs, KV, Sc, g, Rg, R, ldq, ldkv, dp, TQ, rep, nq, nbk, i_lo, j0, km, tid, nth);
			else if (kt == 2) swa_qk_tiles<2, 4>(a, Qs, KV, Sc, g, Rg, R, ldq, ldkv, dp, TQ, rep, nq, nbk, i_lo, j0, km, tid, nth);
			else if ((Rg >> 2) * SWA_KB >= nth) swa_qk_tiles<1, 4>(a, Qs, KV, Sc, g, Rg, R, ldq, ldkv, dp, TQ, rep, nq, nbk, i_lo, j0, km, tid, nth);
			else swa_qk_tiles<1, 2>(a, Qs, KV, Sc, g, Rg, R, ldq, ldkv, dp, TQ, rep, nq, nbk, i_lo, j0, km, tid, nth);
		}
		__syncthreads();
		// ---- mix the heads' scores (4 output heads per thread), mask ----
		for (int x = tid; x < SWA_KB * TQ * (Hp >> 2); x += nth) {
			const int hq = x % (Hp >> 2), rest = x / (Hp >> 2), q = rest % TQ, jj = rest / TQ;
			float m4[4] = {0.f, 0.f, 0.f, 0.f};
			const float* srow = Sc + (size_t) jj * R + q;
			if (!a.talk) { // no mixing: every head keeps its own score
#pragma unroll
				for (int u = 0; u < 4; u++) {
					const int h = min(4 * hq + u, H - 1);
					m4[u] = srow[(h / rep) * Rg + (h % rep) * TQ];
				}
			} else
			for (int g = 0; g < H; g++) {
				const float s = srow[(g / rep) * Rg + (g % rep) * TQ];
				const float4 w = *reinterpret_cast<const float4*>(tkT + g * Hp + 4 * hq);
				m4[0] = fmaf(w.x, s, m4[0]); m4[1] = fmaf(w.y, s, m4[1]); m4[2] = fmaf(w.z, s, m4[2]); m4[3] = fmaf(w.w, s, m4[3]);
			}
			const int i = i_lo + q, j = km.pos(j0 + jj);
			const bool seen = q < nq && jj < nbk && j <= i && (a.window >= 0x7fffffff || i - j < a.window || j < a.keep_first);
#pragma unroll
			for (int u = 0; u < 4; u++) {
				const int h = 4 * hq + u;
				if (h < H) Pr[(size_t) jj * R + (h / rep) * Rg + (h % rep) * TQ + q] = seen ? m4[u] : -INFINITY;
			}
		}
		__syncthreads();
		// ---- online softmax, a warp per (head, query) row; lane = key ----
		for (int x = warp; x < H * TQ; x += nw) {
			const int h = x / TQ, q = x % TQ, row = (h / rep) * Rg + (h % rep) * TQ + q;
			const float s = Pr[(size_t) lane * R + row]; // SWA_KB == 32
			const float bm = warp_max(s);
			const float m_old = mrun[row], m_new = fmaxf(m_old, bm);
			const float p = (m_new == -INFINITY) ? 0.f : expf(s - m_new);
			const float ps = warp_sum(p);
			Pr[(size_t) lane * R + row] = p;
			if (lane == 0) {
				const float al = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
				alpha[row] = al;
				mrun[row] = m_new;
				lrun[row] = lrun[row] * al + ps;
			}
		}
		// ---- O <- alpha O + P^T V, one kv group at a time ----
		for (int g = 0; g < G; g++) {
			__syncthreads(); // probabilities written; the last reader of KV is done
			swa_load_tile(KV, ldkv, vc, a.ldv ? a.ldv : G * dv, g * dv, dv, dvp, j0, nbk, km, tid, nth);
			__syncthreads();
			if ((Rg >> 2) * (dvp >> 2) >= nth) swa_pv_tiles<4>(Pr, KV, O, alpha, g, Rg, R, ldkv, dvp, tid, nth);
			else swa_pv_tiles<2>(Pr, KV, O, alpha, g, Rg, R, ldkv, dvp, tid, nth);
		}
	}
	__syncthreads();
	for (int x = tid; x < nq * H * dv; x += nth) {
		const int c = x % dv, h = (x / dv) % H, q = x / (dv * H), row = (h / rep) * Rg + (h % rep) * TQ + q;
		const int t = t0 + q;
		const float acc = O[(size_t) row * dvp + c];
		if (a.n_splits == 1) {
			float o = swa_finish(a, h, acc, lrun[row], mrun[row]);
			if (a.gate) o *= sigmoidf_(a.gate[(size_t) t * a.ldg + a.g_off + h * dv + c]);
			a.out[(size_t) t * (a.ldo ? a.ldo : H * dv) + h * dv + c] = o;
		} else a.part_o[((size_t) t * a.n_splits + sp) * (H * dv) + h * dv + c] = acc;
	}
	if (a.n_splits > 1)
		for (int x = tid; x < nq * H; x += nth) {
			const int h = x % H, q = x / H, row = (h / rep) * Rg + (h % rep) * TQ + q;
			float* pml = a.part_ml + ((size_t) (t0 + q) * a.n_splits + sp) * (H * 2);
			pml[2 * h] = mrun[row];
			pml[2 * h + 1] = lrun[row];
		}
	if (a.n_splits > 1 && a.tickets) swa_join_last(a, blockIdx.x, t0, nq, tid, nth);
}

// ---- gated linear recurrence (HGRN2) --------------------------------------------------------------------------------------------
struct Hgrn2Args {
	const float* proj; // (T, ld): per head h, q at q_off + h * d, forget pre-activation at f_off + h * d, v at v_off + h * dv
	int ld, q_off, f_off, v_off;
	int H, d, dv;
	const float* f_bias; // (H * d) or NULL
	const float* lower;  // (H * d) lower bound of the forget gate, or NULL (0)
	const float* norm_w; // (dv) plain weight of the per-head RMS norm of o, or NULL (no norm)
	float eps;
	float* state;        // (H, d, dv) fp32, carried between steps
	const SeqStep* step;
	float* out;          // (T, H * dv)
	int max_rows;        // most tokens a step can bring (the launch sizes its shared memory by it)
	int activated;       // 1: proj already holds the forget gate and silu(q) (the producing product's epilogue applied them)
	// Retention: with `decay` set the recurrence is S_t = decay[h] S_{t-1} + (k_scale k_t) v_t^T, o_t = S_t^T q_t: one fixed decay per head, keys
	// of their own at k_off + h * d, q taken as it is (f_off, f_bias, lower and activated are not read)
	const float* decay;  // (H) or NULL
	int k_off;
	float k_scale;
	int norm_plain;      // 1: o over its root mean square with no weight (norm_w NULL)
	const float* gate;   // (T, ldg): o <- o * silu(gate[t, g_off + h * dv + c]) after the norm; NULL: none
	int ldg, g_off;
	// Keyed modes: S_t = diag(f_t) S_{t-1} + (s_t k_t) v_t^T, o_t = S_t^T (q_scale q_t) + skip[h] v_t, with q and k taken as they are from
	// q_off / k_off + (h / qk_rep) * d (qk_rep neighbouring heads share them; 0: 1).
	//   keyed 1: one decay per key channel, ready-made at f_off + h * d + i; s = 1                                  (gated linear attention)
	//   keyed 2: one step size per head and token, dt = softplus(proj[dt_off + h] + dt_bias[h]); f = exp(-exp(A_log[h]) dt) on every
	//            channel, s = dt                                                                                  (state-space duality)
	int keyed;
	int qk_rep;
	float q_scale;       // 0: 1
	int dt_off;
	const float *dt_bias, *A_log; // (H)
	const float* skip;   // (H) or NULL
};
constexpr int HG_TC = 8; // tokens staged at a time
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }
// decay, key factor and query of channel i of head h for one token's row, in a keyed mode
__device__ __forceinline__ void hgrn2_keyed(const Hgrn2Args& a, int h, float f_raw, float k_raw, float q_raw, float& f, float& g, float& q) {
	float s = 1.f;
	f = f_raw;
	if (a.keyed == 2) {
		s = softplusf_(f_raw + a.dt_bias[h]);
		f = expf(-expf(a.A_log[h]) * s);
	}
	g = k_raw * s;
	q = a.q_scale != 0.f ? q_raw * a.q_scale : q_raw;
}

static __global__ void hgrn2_kernel(Hgrn2Args a) {
	extern __shared__ float sm[];
	const int d = a.d, dv = a.dv, h = blockIdx.x, tid = threadIdx.x, nth = blockDim.x;
	float* S = sm;                  // d * dv
	float* fch = S + (size_t) d * dv; // TC * d
	float* qch = fch + HG_TC * d;   // TC * d
	float* gch = qch + HG_TC * d;   // TC * d  what multiplies v: 1 - f, or the key
	float* och = gch + HG_TC * d;   // TC * dv
	float* st = a.state + (size_t) h * d * dv;
	for (int x = tid; x < d * dv; x += nth) S[x] = st[x];
	const int T = a.step->n;
	for (int t0 = 0; t0 < T; t0 += HG_TC) {
		const int nt = min(HG_TC, T - t0);
		__syncthreads();
		for (int x = tid; x < nt * d; x += nth) {
			const int tt = x / d, i = x % d;
			const float* row = a.proj + (size_t) (t0 + tt) * a.ld;
			if (a.keyed) {
				const int hk = h / max(a.qk_rep, 1);
				hgrn2_keyed(a, h, a.keyed == 2 ? row[a.dt_off + h] : row[a.f_off + h * d + i], row[a.k_off + hk * d + i], row[a.q_off + hk * d + i], fch[x], gch[x], qch[x]);
				continue;
			}
			const float zq = row[a.q_off + h * d + i];
			if (a.decay) {
				fch[x] = a.decay[h];
				gch[x] = row[a.k_off + h * d + i] * a.k_scale;
				qch[x] = zq;
				continue;
			}
			const float z = row[a.f_off + h * d + i] + (a.f_bias && !a.activated ? a.f_bias[h * d + i] : 0.f);
			const float lo = a.lower ? a.lower[h * d + i] : 0.f;
			fch[x] = a.activated ? z : lo + (1.f - lo) * sigmoidf_(z);
			gch[x] = 1.f - fch[x];
			qch[x] = a.activated ? zq : zq * sigmoidf_(zq);
		}
		__syncthreads();
		for (int c = tid; c < dv; c += nth) {
			for (int tt = 0; tt < nt; tt++) {
				const float v = a.proj[(size_t) (t0 + tt) * a.ld + a.v_off + h * dv + c];
				const float* f = fch + tt * d;
				const float* q = qch + tt * d;
				const float* gk = gch + tt * d;
				float o = 0.f;
				for (int i = 0; i < d; i++) {
					const float fi = f[i];
					const float s = fmaf(fi, S[(size_t) i * dv + c], gk[i] * v);
					S[(size_t) i * dv + c] = s;
					o = fmaf(s, q[i], o);
				}
				och[tt * dv + c] = a.skip ? fmaf(a.skip[h], v, o) : o;
			}
		}
		__syncthreads();
		for (int tt = tid >> 5; tt < nt; tt += nth >> 5) {
			const int lane = tid & 31;
			float r = 1.f;
			if (a.norm_w || a.norm_plain) {
				float ss = 0.f;
				for (int c = lane; c < dv; c += 32) ss = fmaf(och[tt * dv + c], och[tt * dv + c], ss);
				ss = warp_sum(ss);
				r = 1.f / sqrtf(ss / (float) dv + a.eps);
			}
			float* orow = a.out + (size_t) (t0 + tt) * (a.H * dv) + h * dv;
			const float* grow = a.gate ? a.gate + (size_t) (t0 + tt) * a.ldg + a.g_off + h * dv : nullptr;
			for (int c = lane; c < dv; c += 32) {
				float o = och[tt * dv + c] * r * (a.norm_w ? a.norm_w[c] : 1.f);
				if (grow) o *= grow[c] * sigmoidf_(grow[c]);
				orow[c] = o;
			}
		}
	}
	__syncthreads();
	for (int x = tid; x < d * dv; x += nth) st[x] = S[x];
}
inline size_t hgrn2_smem_bytes(int d, int dv) { return sizeof(float) * ((size_t) d * dv + 3 * (size_t) HG_TC * d + (size_t) HG_TC * dv); }

// ---- the same recurrence, the state's columns spread over warps, CTAs and a thread-block cluster ---------------------------------
// Column c of a head's state evolves on its own: S[:, c] <- f .* S[:, c] + (1 - f) v[c], o[c] = q . S[:, c].  A warp owns HG_CW columns
// with the d channels across its lanes (DPL per lane) in registers; a CTA owns warps x HG_CW columns; the CTAs of one head form a
// cluster (grid.x = cluster size <= 8).  Tokens are staged HG_TT at a time (activations applied once per CTA); the lanes' partial dot
// products of a tile (HG_TT x HG_CW = 32 values) are summed with one transposed butterfly (31 shuffles instead of 160).  The RMS norm
// over a head's dv columns needs every CTA's share: each keeps its per-token sums of squares in shared memory, and after one cluster
// barrier reads the others' through distributed shared memory and scales the rows it wrote.
constexpr int HG_CW = 4, HG_TT = 8;

// v[k] of every lane -> lane k gets the sum over lanes of v[k]
__device__ __forceinline__ float warp_sum_transposed32(float (&v)[32], int lane) {
#pragma unroll
	for (int s = 16; s >= 1; s >>= 1) {
		const bool up = (lane & s) != 0;
#pragma unroll
		for (int k = 0; k < s; k++) {
			const float send = up ? v[k] : v[k + s];
			const float keep = up ? v[k + s] : v[k];
			v[k] = keep + __shfl_xor_sync(0xffffffffu, send, s);
		}
	}
	return v[0];
}

template <int DPL, int KEYED>
__global__ void hgrn2_cols_kernel(Hgrn2Args a) {
	namespace cg = cooperative_groups;
	cg::cluster_group cluster = cg::this_cluster();
	extern __shared__ float sm[];
	constexpr int DP = DPL * 32;
	constexpr int NPF = HG_TT * DP / 128; // (channel, token) pairs a thread of the smallest CTA stages per tile
	const int d = a.d, dv = a.dv, h = blockIdx.y, tid = threadIdx.x, nth = blockDim.x, lane = tid & 31, warp = tid >> 5, nw = nth >> 5;
	const int cpb = nw * HG_CW, c_blk = blockIdx.x * cpb, c0 = c_blk + warp * HG_CW;
	const int tile_floats = 3 * HG_TT * DP + HG_TT * cpb; // f | 1 - f | silu(q) | v of one tile
	float* och = sm + 2 * tile_floats; // HG_TT * cpb  o before the norm
	float* ssq = och + HG_TT * cpb;    // max_rows     this CTA's share of sum_c o[t][c]^2
	float* st = a.state + (size_t) h * d * dv;
	const int T = min(a.step->n, a.max_rows);
	float S[HG_CW][DPL];
#pragma unroll
	for (int cc = 0; cc < HG_CW; cc++)
#pragma unroll
		for (int k = 0; k < DPL; k++) {
			const int i = lane + 32 * k, c = c0 + cc;
			S[cc][k] = (i < d && c < dv) ? st[(size_t) i * dv + c] : 0.f;
		}
	// The next tile's inputs travel through registers while this tile is scanned: raw loads are issued before the scan, the
	// activations (unless the producer already applied them) and the stores to the other buffer come after it.
	float rf[NPF], rq[NPF], rk[KEYED ? NPF : 1], rv = 0.f;
	const int hk = KEYED ? h / max(a.qk_rep, 1) : h;
	auto fetch = [&](int t0) {
		const int nt = min(HG_TT, T - t0);
#pragma unroll
		for (int u = 0; u < NPF; u++) {
			const int x = tid + u * nth, tt = x / DP, i = x % DP;
			rf[u] = 0.f; rq[u] = 0.f;
			if (KEYED) rk[KEYED ? u : 0] = 0.f;
			if (x < HG_TT * DP && tt < nt && i < d) {
				const float* row = a.proj + (size_t) (t0 + tt) * a.ld;
				if (KEYED) {
					rf[u] = a.keyed == 2 ? row[a.dt_off + h] : row[a.f_off + h * d + i];
					rk[KEYED ? u : 0] = row[a.k_off + hk * d + i];
					rq[u] = row[a.q_off + hk * d + i];
				} else {
					rf[u] = row[(a.decay ? a.k_off : a.f_off) + h * d + i];
					rq[u] = row[a.q_off + h * d + i];
				}
			}
		}
		const int tt = tid / cpb, c = c_blk + tid % cpb; // nth == HG_TT * cpb
		rv = (tt < nt && c < dv) ? a.proj[(size_t) (t0 + tt) * a.ld + a.v_off + h * dv + c] : 0.f;
	};
	auto stage = [&](float* buf, int t0) {
		const int nt = min(HG_TT, T - t0);
#pragma unroll
		for (int u = 0; u < NPF; u++) {
			const int x = tid + u * nth, tt = x / DP, i = x % DP;
			if (x < HG_TT * DP) {
				float f = 0.f, g = 0.f, q = 0.f;
				if (tt < nt && i < d) {
					if (KEYED) hgrn2_keyed(a, h, rf[u], rk[KEYED ? u : 0], rq[u], f, g, q);
					else if (a.decay) { f = a.decay[h]; g = rf[u] * a.k_scale; q = rq[u]; }
					else {
						if (a.activated) { f = rf[u]; q = rq[u]; }
						else {
							const float lo = a.lower ? a.lower[h * d + i] : 0.f;
							f = lo + (1.f - lo) * sigmoidf_(rf[u] + (a.f_bias ? a.f_bias[h * d + i] : 0.f));
							q = rq[u] * sigmoidf_(rq[u]);
						}
						g = 1.f - f;
					}
				}
				buf[x] = f; buf[HG_TT * DP + x] = g; buf[2 * HG_TT * DP + x] = q;
			}
		}
		buf[3 * HG_TT * DP + tid] = rv;
	};
	if (T > 0) {
		fetch(0);
		stage(sm, 0);
	}
	__syncthreads();
	int cur = 0;
	for (int t0 = 0; t0 < T; t0 += HG_TT, cur ^= 1) {
		const int nt = min(HG_TT, T - t0);
		const float* fch = sm + cur * tile_floats;
		const float* gch = fch + HG_TT * DP;
		const float* qch = gch + HG_TT * DP;
		const float* vch = qch + HG_TT * DP;
		const bool more = t0 + HG_TT < T;
		if (more) fetch(t0 + HG_TT);
		float p[HG_TT * HG_CW];
#pragma unroll
		for (int tt = 0; tt < HG_TT; tt++) {
#pragma unroll
			for (int cc = 0; cc < HG_CW; cc++) p[tt * HG_CW + cc] = 0.f;
			if (tt < nt) {
				float v[HG_CW];
#pragma unroll
				for (int cc = 0; cc < HG_CW; cc++) v[cc] = vch[tt * cpb + warp * HG_CW + cc];
#pragma unroll
				for (int k = 0; k < DPL; k++) {
					const float fi = fch[tt * DP + lane + 32 * k], gi = gch[tt * DP + lane + 32 * k], qi = qch[tt * DP + lane + 32 * k];
#pragma unroll
					for (int cc = 0; cc < HG_CW; cc++) {
						S[cc][k] = fmaf(fi, S[cc][k], gi * v[cc]);
						p[tt * HG_CW + cc] = fmaf(S[cc][k], qi, p[tt * HG_CW + cc]);
					}
				}
			}
		}
		float o = warp_sum_transposed32(p, lane); // lane = tt * HG_CW + cc
		if (KEYED && a.skip) o = fmaf(a.skip[h], vch[(lane / HG_CW) * cpb + warp * HG_CW + lane % HG_CW], o);
		och[(lane / HG_CW) * cpb + warp * HG_CW + lane % HG_CW] = o;
		if (more) stage(sm + (cur ^ 1) * tile_floats, t0 + HG_TT);
		__syncthreads();
		for (int tt = warp; tt < nt; tt += nw) {
			float ss = 0.f;
			float* orow = a.out + (size_t) (t0 + tt) * (a.H * dv) + h * dv;
			for (int cc = lane; cc < cpb; cc += 32)
				if (c_blk + cc < dv) {
					const float x = och[tt * cpb + cc];
					orow[c_blk + cc] = x;
					ss = fmaf(x, x, ss);
				}
			ss = warp_sum(ss);
			if (lane == 0) ssq[t0 + tt] = ss;
		}
		__syncthreads(); // och is free for the next tile
	}
#pragma unroll
	for (int cc = 0; cc < HG_CW; cc++)
#pragma unroll
		for (int k = 0; k < DPL; k++) {
			const int i = lane + 32 * k, c = c0 + cc;
			if (i < d && c < dv) st[(size_t) i * dv + c] = S[cc][k];
		}
	const bool normed = a.norm_w || a.norm_plain;
	if (!normed && !a.gate) return; // uniform over the cluster: nobody waits
	cluster.sync();
	const unsigned nb = cluster.num_blocks();
	for (int t = warp; t < T; t += nw) {
		float r = 1.f;
		if (normed) {
			float tot = lane < (int) nb ? cluster.map_shared_rank(ssq, lane)[t] : 0.f;
			tot = warp_sum(tot);
			r = 1.f / sqrtf(tot / (float) dv + a.eps);
		}
		float* orow = a.out + (size_t) t * (a.H * dv) + h * dv;
		const float* grow = a.gate ? a.gate + (size_t) t * a.ldg + a.g_off + h * dv : nullptr;
		for (int cc = lane; cc < cpb; cc += 32)
			if (c_blk + cc < dv) {
				float o = orow[c_blk + cc] * r * (a.norm_w ? a.norm_w[c_blk + cc] : 1.f);
				if (grow) o *= grow[c_blk + cc] * sigmoidf_(grow[c_blk + cc]);
				orow[c_blk + cc] = o;
			}
	}
	cluster.sync(); // no CTA leaves while another still reads its sums
}
inline size_t hgrn2_cols_smem_bytes(int dpl, int warps, int max_rows) {
	return sizeof(float) * (2 * (3 * (size_t) HG_TT * dpl * 32 + (size_t) HG_TT * warps * HG_CW) + (size_t) HG_TT * warps * HG_CW + (size_t) max_rows);
}

// ---- y = 1/2 (rmsnorm(a) wa + rmsnorm(b) wb), layer scale, hyper-connection write -------------------------------------------------
// The read of the sublayer that follows can ride along: with next.h set, the streams just written are combined with next.a, RMS-normed
// with next.w and stored to next.h (what hc_norm_kernel would do in a launch of its own; the arithmetic is the same, in the same order).
struct NextRead {
	const float* a = nullptr; // (S) coefficients, NULL: ones
	const float* w = nullptr; // (width) norm weight
	int one_plus = 1;
	float* h = nullptr;       // (T, width), NULL: nothing rides along
};
template <int SS>
__global__ void dual_norm_hc_kernel(const float* __restrict__ A, const float* __restrict__ B, const float* __restrict__ wa, const float* __restrict__ wb,
                                    float eps, int width, RowsEpi e, NextRead next) {
	extern __shared__ float sm[];
	__shared__ float hm[MAX_STREAMS * MAX_STREAMS], ho[MAX_STREAMS], an[MAX_STREAMS];
	float* red = sm;      // 33
	float* un = sm + 33;  // width, when next.h is set
	const int t = blockIdx.x, tid = threadIdx.x, nth = blockDim.x, S = e.S;
	for (int x = tid; x < S * S; x += nth) hm[x] = e.hmix ? e.hmix[x] : (x / S == x % S ? 1.f : 0.f);
	if (tid < S) ho[tid] = e.hout ? e.hout[tid] : 1.f;
	if (tid < S) an[tid] = next.a ? next.a[tid] : 1.f;
	float ssn = 0.f;
	// four columns per thread at a time, loads first (see hc_norm_kernel)
	float sa = 0.f, sb = 0.f;
	for (int c0 = 0; c0 < width; c0 += 4 * nth) {
		float x[4], y[4];
#pragma unroll
		for (int k = 0; k < 4; k++) {
			const int c = c0 + k * nth + tid;
			x[k] = c < width ? A[(size_t) t * width + c] : 0.f;
			y[k] = c < width ? B[(size_t) t * width + c] : 0.f;
		}
#pragma unroll
		for (int k = 0; k < 4; k++) {
			sa = fmaf(x[k], x[k], sa);
			sb = fmaf(y[k], y[k], sb);
		}
	}
	const float ra = 1.f / sqrtf(block_sum(sa, red) / (float) width + eps);
	const float rb = 1.f / sqrtf(block_sum(sb, red) / (float) width + eps); // block_sum's barriers also publish hm / ho
	for (int c0 = 0; c0 < width; c0 += 4 * nth) {
		float x[4], y[4], wx[4], wy[4], sc[4], old[4][SS];
#pragma unroll
		for (int k = 0; k < 4; k++) {
			const int c = c0 + k * nth + tid;
			const bool in = c < width;
			x[k] = in ? A[(size_t) t * width + c] : 0.f;
			y[k] = in ? B[(size_t) t * width + c] : 0.f;
			wx[k] = in ? wa[c] : 0.f;
			wy[k] = in ? wb[c] : 0.f;
			sc[k] = (in && e.scale) ? e.scale[c] : 1.f;
#pragma unroll
			for (int s = 0; s < SS; s++) old[k][s] = (in && s < S) ? e.xs[(size_t) s * e.stream_stride + (size_t) t * width + c] : 0.f;
		}
#pragma unroll
		for (int k = 0; k < 4; k++) {
			const int c = c0 + k * nth + tid;
			if (c >= width) continue;
			const float v = 0.5f * (x[k] * ra * wx[k] + y[k] * rb * wy[k]);
			const float yv = e.scale ? sc[k] * v : v;
			float u2 = 0.f;
#pragma unroll
			for (int q = 0; q < SS; q++)
				if (q < S) {
					float acc = 0.f;
					if (e.hmix) {
#pragma unroll
						for (int s2 = 0; s2 < SS; s2++)
							if (s2 < S) acc = fmaf(hm[s2 * S + q], old[k][s2], acc);
					} else {
#pragma unroll
						for (int s2 = 0; s2 < SS; s2++)
							if (s2 == q) acc = old[k][s2];
					}
					const float nv = fmaf(ho[q], yv, acc);
					e.xs[(size_t) q * e.stream_stride + (size_t) t * width + c] = nv;
					u2 = next.a ? fmaf(an[q], nv, u2) : u2 + nv;
				}
			if (next.h) {
				un[c] = u2;
				ssn = fmaf(u2, u2, ssn);
			}
		}
	}
	if (!next.h) return;
	const float rn = 1.f / sqrtf(block_sum(ssn, red) / (float) width + eps);
	for (int c0 = 0; c0 < width; c0 += 4 * nth) {
		float wv[4];
#pragma unroll
		for (int k = 0; k < 4; k++) {
			const int c = c0 + k * nth + tid;
			wv[k] = c < width ? next.w[c] : 0.f;
		}
#pragma unroll
		for (int k = 0; k < 4; k++) {
			const int c = c0 + k * nth + tid;
			if (c < width) next.h[(size_t) t * width + c] = un[c] * rn * (next.one_plus ? 1.f + wv[k] : wv[k]); // un[c]: written by this thread
		}
	}
}

// ---- host-side launchers (shared by the model families and the op-level entry points) ------------------------------------------
static inline int launch_check(const char* what) {
	const cudaError_t e = cudaGetLastError();
	if (e != cudaSuccess) return set_error(XALM_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
	return XALM_OK;
}
static inline int norm_threads(int width) { return width >= 1024 ? 256 : width >= 256 ? 128 : 64; }

// out(T,N) = A(T,K) . W(N,K)^T with epilogue e, IEEE fp32 arithmetic; W is bf16 or fp32
// batch > 1: that many products in one launch, operands and output advancing by e.batch_a / batch_w / batch_o per product
static inline int launch_rows(const float* A, int lda, const void* W, bool w_bf16, int T, int N, int K, const RowsEpi& e, cudaStream_t s, int batch = 1) {
	if (T <= 4) {
		const int pairs = (N + 1) / 2;
		int ks = 1; // warps per column pair: enough CTAs for two per SM, each slice of K at least 256 long
		while (ks < 8 && (pairs * ks + 7) / 8 * batch < 296 && K >= 512 * ks) ks *= 2;
		const dim3 grid((pairs * ks + 7) / 8, 1, batch);
#define XALM_ROWS_MATVEC(WT_, TB_)                                                                                                   \
	do {                                                                                                                             \
		if (ks == 1) rows_matvec_kernel<WT_, TB_, 1><<<grid, 256, 0, s>>>(A, lda, (const WT_*) W, T, N, K, e);                       \
		else if (ks == 2) rows_matvec_kernel<WT_, TB_, 2><<<grid, 256, 0, s>>>(A, lda, (const WT_*) W, T, N, K, e);                  \
		else if (ks == 4) rows_matvec_kernel<WT_, TB_, 4><<<grid, 256, 0, s>>>(A, lda, (const WT_*) W, T, N, K, e);                  \
		else rows_matvec_kernel<WT_, TB_, 8><<<grid, 256, 0, s>>>(A, lda, (const WT_*) W, T, N, K, e);                               \
	} while (0)
		if (w_bf16) {
			if (T == 1) XALM_ROWS_MATVEC(__nv_bfloat16, 1);
			else XALM_ROWS_MATVEC(__nv_bfloat16, 4);
		} else {
			if (T == 1) XALM_ROWS_MATVEC(float, 1);
			else XALM_ROWS_MATVEC(float, 4);
		}
#undef XALM_ROWS_MATVEC
	} else {
		const dim3 grid((N + 63) / 64, (T + 63) / 64, batch);
		if (w_bf16) rows_gemm_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(A, lda, (const __nv_bfloat16*) W, T, N, K, e);
		else rows_gemm_kernel<float><<<grid, 256, 0, s>>>(A, lda, (const float*) W, T, N, K, e);
	}
	return launch_check("row product");
}

// Kernels whose shared memory can pass 48 KB raise their limit once per process (these families run on one device).  A family calls
// the prepare functions when it finalizes, so that no attribute changes while a step is captured into a graph.
static inline int hc_norm_prepare(int width) {
	static bool raised = false;
	if ((size_t) (width + 33) * 4 > 48 * 1024 && !raised) {
		XALM_CUDA_CHECK(cudaFuncSetAttribute(hc_norm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
		XALM_CUDA_CHECK(cudaFuncSetAttribute(hc_norm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
		XALM_CUDA_CHECK(cudaFuncSetAttribute(hc_norm_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
		XALM_CUDA_CHECK(cudaFuncSetAttribute(hc_norm_kernel<MAX_STREAMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
		raised = true;
	}
	return XALM_OK;
}
static inline int swa_prepare(int H, int d, int dv) { // before any launch (and outside a stream capture): the kernels may ask for up to 200 KB
	static bool raised = false;
	(void) H; (void) d; (void) dv;
	if (!raised) {
		XALM_CUDA_CHECK(cudaFuncSetAttribute(swa_attn_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
		XALM_CUDA_CHECK(cudaFuncSetAttribute(swa_attn_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
		raised = true;
	}
	return XALM_OK;
}
static inline int hgrn2_prepare(int d, int dv) {
	static bool raised = false;
	if (hgrn2_smem_bytes(d, dv) > 48 * 1024 && !raised) {
		XALM_CUDA_CHECK(cudaFuncSetAttribute(hgrn2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
		raised = true;
	}
	return XALM_OK;
}

// ---- grouped RMS norm of a sublayer's output, residual add, depth-weighted average ------------------------------------------------
// For designs that norm what a sublayer returns and not what it reads:  v = x_in + gnorm(y) * w, where gnorm splits the row into
// `groups` equal consecutive parts and divides each by its own sqrt(mean(part^2) + eps).  Along for the ride, because each is one more
// pass over the same row otherwise:
//   * y may come in `parts` rows per token that are first summed with weights part_w (the chosen experts of a mixture, in slot order:
//     a fixed order, so the sum is the same bits every run);
//   * the depth-weighted average: with hist holding the earlier layers' results X_0 .. X_{n_hist-1} for this pass and v being X_{n_hist},
//     avg_out = sum_j dwa[j] X_j is what the next layer reads;
//   * keep_out: a copy of what goes on to the next layer, for readers outside the model.
struct GroupNormArgs {
	const float* y = nullptr;      // (rows * parts, ldy)
	int ldy = 0, parts = 1;
	const float* part_w = nullptr; // (rows, parts), or NULL: parts == 1 with weight 1
	const int* part_row = nullptr; // (rows, parts) row of y that holds part k of token t, or NULL: t * parts + k
	const float* w = nullptr;      // (width)
	int groups = 1, width = 0;
	float eps = 1e-5f;
	const float* x_in = nullptr;   // (rows, width) or NULL: no residual (the model's final norm)
	float* x_out = nullptr;        // (rows, width); may be x_in
	const float* hist = nullptr;   // (n_hist, hist_stride) earlier results of this pass, or NULL
	size_t hist_stride = 0;
	int n_hist = 0;
	const float* dwa = nullptr;    // (n_hist + 1)
	float* avg_out = nullptr;      // (rows, width)
	float* keep_out = nullptr;     // (rows, width) or NULL
	const float* gate = nullptr;   // (rows, ldg) or NULL: y <- y * silu(gate) before the norm (a gated recurrence whose norm follows the gate)
	int ldg = 0;
	float out_scale = 0.f;         // multiplies the normed, weighted row (0: 1)
	int ld_out = 0;                // elements between rows of x_out (0: width): the result may be a run of columns of a wider buffer
};
static __global__ void group_norm_residual_kernel(GroupNormArgs a) {
	extern __shared__ float sm[];
	float* u = sm;               // width
	float* rinv = sm + a.width;  // groups
	const int t = blockIdx.x, tid = threadIdx.x, nth = blockDim.x, lane = tid & 31, warp = tid >> 5, nw = nth >> 5;
	const int W = a.width, gs = W / a.groups;
	// four columns per thread at a time, every load of the four issued before the first use: a one-token step runs one CTA of this kernel,
	// and its time is the number of dependent trips to memory
	for (int c0 = tid; c0 < W; c0 += 4 * nth) {
		float v[4];
#pragma unroll
		for (int k = 0; k < 4; k++) {
			const int c = c0 + k * nth;
			v[k] = 0.f;
			if (c < W) {
				if (a.part_w) {
					for (int p = 0; p < a.parts; p++) {
						const size_t pk = (size_t) t * a.parts + p;
						v[k] = fmaf(a.part_w[pk], a.y[(a.part_row ? (size_t) a.part_row[pk] : pk) * a.ldy + c], v[k]);
					}
				} else v[k] = a.y[(size_t) t * a.ldy + c];
				if (a.gate) {
					const float z = a.gate[(size_t) t * a.ldg + c];
					v[k] *= z * sigmoidf_(z);
				}
			}
		}
#pragma unroll
		for (int k = 0; k < 4; k++)
			if (c0 + k * nth < W) u[c0 + k * nth] = v[k];
	}
	__syncthreads();
	for (int g = warp; g < a.groups; g += nw) {
		float ss = 0.f;
		for (int c = lane; c < gs; c += 32) ss = fmaf(u[g * gs + c], u[g * gs + c], ss);
		ss = warp_sum(ss);
		if (lane == 0) rinv[g] = 1.f / sqrtf(ss / (float) gs + a.eps);
	}
	__syncthreads();
	for (int c0 = tid; c0 < W; c0 += 4 * nth) {
		float wv[4], xi[4], acc[4];
#pragma unroll
		for (int k = 0; k < 4; k++) {
			const int c = c0 + k * nth;
			const bool in = c < W;
			wv[k] = in ? a.w[c] : 0.f;
			xi[k] = (in && a.x_in) ? a.x_in[(size_t) t * W + c] : 0.f;
			acc[k] = 0.f;
		}
		if (a.dwa)
			for (int j = 0; j < a.n_hist; j++) {
				const float cj = a.dwa[j];
				float hv[4];
#pragma unroll
				for (int k = 0; k < 4; k++) hv[k] = c0 + k * nth < W ? a.hist[(size_t) j * a.hist_stride + (size_t) t * W + c0 + k * nth] : 0.f;
#pragma unroll
				for (int k = 0; k < 4; k++) acc[k] = fmaf(cj, hv[k], acc[k]);
			}
#pragma unroll
		for (int k = 0; k < 4; k++) {
			const int c = c0 + k * nth;
			if (c >= W) continue;
			const size_t at = (size_t) t * W + c;
			float v = u[c] * rinv[c / gs] * wv[k];
			if (a.out_scale != 0.f) v *= a.out_scale;
			if (a.x_in) v += xi[k];
			a.x_out[a.ld_out ? (size_t) t * a.ld_out + c : at] = v;
			if (a.dwa) {
				v = fmaf(a.dwa[a.n_hist], v, acc[k]);
				a.avg_out[at] = v;
			}
			if (a.keep_out) a.keep_out[at] = v;
		}
	}
}
static inline size_t group_norm_smem(int width, int groups) { return (size_t) (width + groups) * 4; }
static inline int group_norm_prepare(int width, int groups) {
	static bool raised = false;
	if (group_norm_smem(width, groups) > 48 * 1024 && !raised) {
		XALM_CUDA_CHECK(cudaFuncSetAttribute(group_norm_residual_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
		raised = true;
	}
	return XALM_OK;
}
static inline int launch_group_norm(const GroupNormArgs& a, int rows, cudaStream_t s) {
	if (a.groups <= 0 || a.width % a.groups) return set_error(XALM_ERR_INVALID, "group norm: %d groups do not divide a row of %d", a.groups, a.width);
	group_norm_residual_kernel<<<rows, norm_threads(a.width), group_norm_smem(a.width, a.groups), s>>>(a);
	return launch_check("group_norm_residual");
}

// ---- after the q | k | v projection of an attention layer: bias, rotary positions, RMS norms without weight, cache write ------------
// One warp per head of a token.  Query heads are rewritten in place; key and value heads go to the cache slot of the token's position
// (SwaKeys layout: the first keep_first positions in slots of their own, the rest in a ring).  Rotation: the first 2 * rot_half
// dimensions of a query / key head, dimension i paired with i + rot_half, angle = position * freq[i] in fp32 (sincosf).  The norms
// (x / sqrt(mean(x^2) + eps) over the head, no weight) come after the rotation; each is optional.
struct QkvPostArgs {
	float* proj; // (T, ld)
	int ld, q_off, k_off, v_off;
	int H, G, d, dv;
	const float *bq, *bk, *bv; // biases of the three projections, or NULL
	const float* freq;         // (rot_half) or NULL
	int rot_half;
	float rot_mag;             // multiplies cos and sin of every turn (a rescaled rotation changes the length of what it turns); 0: 1
	int norm_qk, norm_v;
	float eps;
	void *kc, *vc;
	int cache_f32, keep_first, ring;
	const SeqStep* step;
};
static __global__ void qkv_post_kernel(QkvPostArgs a) {
	extern __shared__ float sm[];
	const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
	const int unit = blockIdx.y * nw + warp;
	if (t >= a.step->n || unit >= a.H + 2 * a.G) return;
	const int wmax = a.d > a.dv ? a.d : a.dv;
	float* x = sm + (size_t) warp * wmax;
	const int pos = a.step->pos0 + t;
	const int kind = unit < a.H ? 0 : unit < a.H + a.G ? 1 : 2; // q, k, v
	const int hd = kind == 0 ? unit : kind == 1 ? unit - a.H : unit - a.H - a.G;
	const int n = kind == 2 ? a.dv : a.d;
	float* src = a.proj + (size_t) t * a.ld + (kind == 0 ? a.q_off : kind == 1 ? a.k_off : a.v_off) + hd * n;
	const float* bias = kind == 0 ? a.bq : kind == 1 ? a.bk : a.bv;
	for (int c = lane; c < n; c += 32) x[c] = src[c] + (bias ? bias[hd * n + c] : 0.f);
	__syncwarp();
	if (kind != 2 && a.freq) {
		const int r = a.rot_half;
		for (int c = lane; c < r; c += 32) {
			float sn, cs;
			sincosf((float) pos * a.freq[c], &sn, &cs);
			if (a.rot_mag != 0.f) { sn *= a.rot_mag; cs *= a.rot_mag; }
			const float p = x[c], q = x[c + r];
			x[c] = p * cs - q * sn;
			x[c + r] = q * cs + p * sn;
		}
		__syncwarp();
	}
	float rs = 1.f;
	if (kind == 2 ? a.norm_v : a.norm_qk) {
		float ss = 0.f;
		for (int c = lane; c < n; c += 32) ss = fmaf(x[c], x[c], ss);
		ss = warp_sum(ss);
		rs = 1.f / sqrtf(ss / (float) n + a.eps);
	}
	if (kind == 0) {
		for (int c = lane; c < n; c += 32) src[c] = x[c] * rs;
		return;
	}
	const int slot = pos < a.keep_first ? pos : a.keep_first + (pos - a.keep_first) % a.ring;
	const size_t at = ((size_t) slot * a.G + hd) * n;
	void* cache = kind == 1 ? a.kc : a.vc;
	if (a.cache_f32)
		for (int c = lane; c < n; c += 32) ((float*) cache)[at + c] = x[c] * rs;
	else
		for (int c = lane; c < n; c += 32) ((__nv_bfloat16*) cache)[at + c] = __float2bfloat16_rn(x[c] * rs);
}
static inline int launch_qkv_post(const QkvPostArgs& a, int rows, cudaStream_t s) {
	const int units = a.H + 2 * a.G, nw = units < 8 ? units : 8, wmax = a.d > a.dv ? a.d : a.dv;
	if ((size_t) nw * wmax * 4 > 48 * 1024) return set_error(XALM_ERR_UNSUPPORTED, "qkv_post: heads of %d do not fit shared memory", wmax);
	qkv_post_kernel<<<dim3(rows, (units + nw - 1) / nw), nw * 32, (size_t) nw * wmax * 4, s>>>(a);
	return launch_check("qkv_post");
}

static inline int launch_embed_pair(const EmbedPairArgs& a, bool w_bf16, int rows, cudaStream_t s) {
	if (a.w && (a.groups <= 0 || a.width % a.groups)) return set_error(XALM_ERR_INVALID, "embedding norm: %d groups do not divide a row of %d", a.groups, a.width);
	if (a.pair && a.buckets <= 0) return set_error(XALM_ERR_INVALID, "pair embedding: %d buckets", a.buckets);
	const size_t smem = (size_t) (a.width + std::max(a.groups, 1)) * 4;
	if (smem > 48 * 1024) return set_error(XALM_ERR_UNSUPPORTED, "embedding: a row of %d does not fit shared memory", a.width);
	if (w_bf16) embed_pair_kernel<__nv_bfloat16><<<rows, norm_threads(a.width), smem, s>>>(a);
	else embed_pair_kernel<float><<<rows, norm_threads(a.width), smem, s>>>(a);
	return launch_check("embed_pair");
}

static inline int launch_rows_epilogue(const float* src, int lds, int T, int N, const RowsEpi& e, cudaStream_t s) {
	const size_t total = (size_t) T * (e.kind == EPI_GLU ? (N + 1) / 2 : N);
	rows_epilogue_kernel<<<(int) std::min<size_t>((total + 255) / 256, 148 * 16), 256, 0, s>>>(src, lds, T, N, e);
	return launch_check("row epilogue");
}

static inline int launch_hc_norm(const float* xs, int S, size_t stream_stride, const float* a, const float* w, int one_plus, float eps, int width, float* h,
                          float* sum_out, int rows, cudaStream_t s) {
	const size_t smem = (size_t) (width + 33) * 4;
	XALM_TRY(hc_norm_prepare(width));
	const int nt = norm_threads(width);
	if (S <= 1) hc_norm_kernel<1><<<rows, nt, smem, s>>>(xs, S, stream_stride, a, w, one_plus, eps, width, h, sum_out);
	else if (S <= 2) hc_norm_kernel<2><<<rows, nt, smem, s>>>(xs, S, stream_stride, a, w, one_plus, eps, width, h, sum_out);
	else if (S <= 4) hc_norm_kernel<4><<<rows, nt, smem, s>>>(xs, S, stream_stride, a, w, one_plus, eps, width, h, sum_out);
	else hc_norm_kernel<MAX_STREAMS><<<rows, nt, smem, s>>>(xs, S, stream_stride, a, w, one_plus, eps, width, h, sum_out);
	return launch_check("hc_norm");
}

// widths whose combined row fits the default 48 KB of dynamic shared memory can carry the next sublayer's read
static inline bool dual_norm_can_carry(int width) { return (size_t) (width + 33) * 4 <= 48 * 1024; }
static inline int launch_dual_norm_hc(const float* A, const float* B, const float* wa, const float* wb, float eps, int width, const RowsEpi& e, int rows,
                                      cudaStream_t s, const NextRead& next = NextRead()) {
	const int nt = norm_threads(width);
	if (next.h && !dual_norm_can_carry(width)) return set_error(XALM_ERR_UNSUPPORTED, "dual_norm_hc: a row of %d does not fit shared memory", width);
	const size_t smem = (size_t) (33 + (next.h ? width : 0)) * 4;
	if (e.S <= 1) dual_norm_hc_kernel<1><<<rows, nt, smem, s>>>(A, B, wa, wb, eps, width, e, next);
	else if (e.S <= 2) dual_norm_hc_kernel<2><<<rows, nt, smem, s>>>(A, B, wa, wb, eps, width, e, next);
	else if (e.S <= 4) dual_norm_hc_kernel<4><<<rows, nt, smem, s>>>(A, B, wa, wb, eps, width, e, next);
	else dual_norm_hc_kernel<MAX_STREAMS><<<rows, nt, smem, s>>>(A, B, wa, wb, eps, width, e, next);
	return launch_check("dual_norm_hc");
}

// Queries per CTA of the tiled kernel: the most (<= 16, <= rows rounded up to a power of two) whose tile leaves room for two CTAs
// per SM, else for one; 0 if not even one query fits (then the one-query kernel above runs).
static inline int swa_pick_tq(int H, int G, int d, int dv, int rows) {
	if (rows <= 4 && swa_smem_bytes(H, d, dv) <= 200 * 1024) return 0; // short steps: the one-query kernel, a CTA per (token, key split)
	int cap = 1;
	while (cap < rows && cap < 16) cap *= 2;
	for (const size_t budget : {(size_t) 110 * 1024, (size_t) 220 * 1024})
		for (int tq = cap; tq >= 1; tq >>= 1)
			if (swa_tile_smem_floats(H, G, d, dv, tq) * 4 <= budget) return tq;
	return 0;
}

// rows: tokens of the step; cache_f32: element type of the ring.  With n_splits > 1 the merge kernel follows.  Returns the number of
// launches through *launches (1 or 2) when it is given.
static inline int launch_swa(SwaArgs a, int rows, bool cache_f32, cudaStream_t s, int* launches = nullptr) {
	// One key/value group, no score mixing, more than a few rows, and all heads together do not fit a CTA's shared memory in the tiled kernel
	// (many heads over a wide latent): the heads run in 2, 4 or 8 launches, each a smaller attention of its own on its share of the query
	// and output columns, with its own slice of the partial buffers and ticket counters.
	if (a.G == 1 && !a.talk && rows > 4 && !a.ldo && !swa_pick_tq(a.H, 1, a.d, a.dv, rows)) {
		for (int nz = 2; nz <= 8; nz *= 2) {
			if (a.H % nz || !swa_pick_tq(a.H / nz, 1, a.d, a.dv, rows)) continue;
			const int Hc = a.H / nz;
			const int cap = a.n_splits > 0 ? rows * a.n_splits : a.part_cap;
			if (launches) *launches = 0;
			for (int z = 0; z < nz; z++) {
				SwaArgs b = a;
				b.H = Hc;
				b.ldo = a.H * a.dv;
				b.q_off = a.q_off + z * Hc * a.d;
				b.g_off = a.g_off + z * Hc * a.dv;
				if (a.sink) b.sink = a.sink + (size_t) z * Hc;
				b.out = a.out + (size_t) z * Hc * a.dv;
				if (a.part_o) b.part_o = a.part_o + (size_t) z * cap * Hc * a.dv;
				if (a.part_ml) b.part_ml = a.part_ml + (size_t) z * cap * Hc * 2;
				if (a.tickets) b.tickets = a.tickets + (size_t) z * rows;
				int one = 1;
				XALM_TRY(launch_swa(b, rows, cache_f32, s, &one));
				if (launches) *launches += one;
			}
			return XALM_OK;
		}
	}
	const int tq = swa_pick_tq(a.H, a.G, a.d, a.dv, rows);
	if (a.n_splits <= 0) { // enough CTAs for two waves, at least two key blocks each
		const int qblocks = tq ? (rows + tq - 1) / tq : rows;
		const long long keys = std::min<long long>((long long) a.ring, (long long) (a.window < 0x7fffffff ? a.window : a.ring) + (tq ? tq : 1)) + a.keep_first;
		int want = std::max(1, 296 / std::max(1, qblocks));
		want = (int) std::min<long long>(want, std::max<long long>(1, tq ? keys / (2 * SWA_KB) : (keys + SWA_KB - 1) / SWA_KB)); // key blocks per CTA: >= 2 (tiled), 1 (one query)
		a.n_splits = (a.part_o && a.part_ml) ? std::max(1, std::min(want, a.part_cap / std::max(1, rows))) : 1;
	}
	if (!tq) a.tickets = nullptr; // the one-query kernel's parts are joined by a kernel of many CTAs: one CTA would take longer than the attention
	if (launches) *launches = a.n_splits > 1 && !a.tickets ? 2 : 1;
	if (tq) {
		a.tq = tq;
		const size_t smem = swa_tile_smem_floats(a.H, a.G, a.d, a.dv, tq) * 4;
		if (smem > 48 * 1024) {
			if (cache_f32) XALM_CUDA_CHECK(cudaFuncSetAttribute(swa_tile_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
			else XALM_CUDA_CHECK(cudaFuncSetAttribute(swa_tile_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
		}
		const dim3 grid((rows + tq - 1) / tq, a.n_splits);
		if (cache_f32) swa_tile_kernel<float><<<grid, 256, smem, s>>>(a);
		else swa_tile_kernel<__nv_bfloat16><<<grid, 256, smem, s>>>(a);
	} else {
		size_t smem = swa_smem_bytes(a.H, a.d, a.dv);
		const bool v_in_k = a.vc == a.kc && (a.ldv ? a.ldv : a.G * a.dv) == (a.ldk ? a.ldk : a.G * a.d) && a.G == 1 && a.dv <= a.d; // as the kernel decides
		const size_t staged = swa_stage_off(a.H, a.d, a.dv) * 4 + swa_stage_bytes(a.G, a.d, a.dv, cache_f32, v_in_k);
		a.stage_off = 0;
		const bool rows16 = ((a.d | a.dv | a.ldk | a.ldv) & 7) == 0 && ((reinterpret_cast<uintptr_t>(a.kc) | reinterpret_cast<uintptr_t>(a.vc)) & 15) == 0;
		if (rows16 && staged <= 200 * 1024) { // rows of whole 16-byte pieces, and room for a key block
			a.stage_off = (int) swa_stage_off(a.H, a.d, a.dv);
			smem = staged;
		}
		XALM_TRY(swa_prepare(a.H, a.d, a.dv));
		if (cache_f32) swa_attn_kernel<float><<<dim3(rows, a.n_splits), 256, smem, s>>>(a);
		else swa_attn_kernel<__nv_bfloat16><<<dim3(rows, a.n_splits), 256, smem, s>>>(a);
	}
	XALM_TRY(launch_check("swa_attn"));
	if (a.n_splits > 1 && !a.tickets) {
		swa_merge_kernel<<<dim3(rows, (a.H * a.dv + 127) / 128), 128, 0, s>>>(a);
		XALM_TRY(launch_check("swa_merge"));
	}
	return XALM_OK;
}

// max_rows: an upper bound of the step's tokens known on the host.  The cluster kernel takes d <= 256 and dv <= 1024; anything else
// (and max_rows beyond its shared memory) runs the one-CTA-per-head kernel.
template <int DPL, int KEYED>
static inline int launch_hgrn2_cols(const Hgrn2Args& a, int warps, int nb, cudaStream_t s) {
	const size_t smem = hgrn2_cols_smem_bytes(DPL, warps, a.max_rows);
	if (smem > 48 * 1024) XALM_CUDA_CHECK(cudaFuncSetAttribute(hgrn2_cols_kernel<DPL, KEYED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = dim3(nb, a.H);
	cfg.blockDim = dim3(warps * 32);
	cfg.dynamicSmemBytes = smem;
	cfg.stream = s;
	cudaLaunchAttribute at[1];
	at[0].id = cudaLaunchAttributeClusterDimension;
	at[0].val.clusterDim.x = nb; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
	cfg.attrs = at;
	cfg.numAttrs = 1;
	const cudaError_t e = cudaLaunchKernelEx(&cfg, hgrn2_cols_kernel<DPL, KEYED>, a);
	if (e != cudaSuccess) return set_error(XALM_ERR_CUDA, "hgrn2 launch failed: %s", cudaGetErrorString(e));
	return XALM_OK;
}

// warps per CTA of the cluster kernel for dv columns: the fewest of 4 .. 32 that keep a head within 8 CTAs
static inline int hgrn2_cols_warps(int dv) {
	int warps = 4;
	while (warps < 32 && (dv + warps * HG_CW - 1) / (warps * HG_CW) > 8) warps *= 2;
	return warps;
}
// registers per thread of the instance that serves dpl channels per lane, as compiled (asked of the runtime once; a table if it will not say)
static inline int hgrn2_cols_regs(int dpl, bool keyed) {
	static int known[2][4] = {};
	const int slot = dpl <= 1 ? 0 : dpl <= 2 ? 1 : dpl <= 4 ? 2 : 3;
	int& r = known[keyed ? 1 : 0][slot];
	if (!r) {
		cudaFuncAttributes at = {};
		cudaError_t e;
		if (keyed) e = slot == 0 ? cudaFuncGetAttributes(&at, hgrn2_cols_kernel<1, 1>) : slot == 1 ? cudaFuncGetAttributes(&at, hgrn2_cols_kernel<2, 1>)
		             : slot == 2 ? cudaFuncGetAttributes(&at, hgrn2_cols_kernel<4, 1>) : cudaFuncGetAttributes(&at, hgrn2_cols_kernel<8, 1>);
		else e = slot == 0 ? cudaFuncGetAttributes(&at, hgrn2_cols_kernel<1, 0>) : slot == 1 ? cudaFuncGetAttributes(&at, hgrn2_cols_kernel<2, 0>)
		         : slot == 2 ? cudaFuncGetAttributes(&at, hgrn2_cols_kernel<4, 0>) : cudaFuncGetAttributes(&at, hgrn2_cols_kernel<8, 0>);
		if (e != cudaSuccess) cudaGetLastError();
		r = e == cudaSuccess && at.numRegs > 0 ? (at.numRegs + 7) / 8 * 8 : slot == 0 ? 64 : slot == 1 ? 112 : slot == 2 ? 128 : 240;
	}
	return r;
}
static inline bool hgrn2_cols_ok(int d, int dv, int max_rows, bool keyed = false) {
	const int warps = hgrn2_cols_warps(dv), nb = (dv + warps * HG_CW - 1) / (warps * HG_CW), dpl = (d + 31) / 32;
	if (dpl > 8) return false;
	const int regs = hgrn2_cols_regs(dpl, keyed); // a CTA's registers must fit one SM's file
	return nb <= 8 && dpl <= 8 && warps * 32 * regs <= 65536 && max_rows > 0 && hgrn2_cols_smem_bytes(dpl <= 1 ? 1 : dpl <= 2 ? 2 : dpl <= 4 ? 4 : 8, warps, max_rows) <= 160 * 1024;
}

static inline int launch_hgrn2(const Hgrn2Args& a, cudaStream_t s) {
	const int warps = hgrn2_cols_warps(a.dv);
	const int nb = (a.dv + warps * HG_CW - 1) / (warps * HG_CW);
	const int dpl = (a.d + 31) / 32;
	if (a.keyed && a.H % std::max(a.qk_rep, 1)) return set_error(XALM_ERR_INVALID, "recurrence: %d heads in groups of %d", a.H, a.qk_rep);
	if (hgrn2_cols_ok(a.d, a.dv, a.max_rows, a.keyed != 0)) {
		if (a.keyed) {
			if (dpl <= 1) return launch_hgrn2_cols<1, 1>(a, warps, nb, s);
			if (dpl <= 2) return launch_hgrn2_cols<2, 1>(a, warps, nb, s);
			if (dpl <= 4) return launch_hgrn2_cols<4, 1>(a, warps, nb, s);
			return launch_hgrn2_cols<8, 1>(a, warps, nb, s);
		}
		if (dpl <= 1) return launch_hgrn2_cols<1, 0>(a, warps, nb, s);
		if (dpl <= 2) return launch_hgrn2_cols<2, 0>(a, warps, nb, s);
		if (dpl <= 4) return launch_hgrn2_cols<4, 0>(a, warps, nb, s);
		return launch_hgrn2_cols<8, 0>(a, warps, nb, s);
	}
	const size_t smem = hgrn2_smem_bytes(a.d, a.dv);
	XALM_TRY(hgrn2_prepare(a.d, a.dv));
	hgrn2_kernel<<<a.H, std::min(1024, (a.dv + 31) / 32 * 32), smem, s>>>(a);
	return launch_check("hgrn2");
}

} // namespace mix
} // namespace xalm
