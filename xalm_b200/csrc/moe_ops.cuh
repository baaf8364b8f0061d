// moe_ops.cuh — a mixture of small gated feed-forward experts, as three mechanisms that another design can use on their own:
//
//   moe_router_kernel   per token: logits z = W_router h in fp32, scores s = sigmoid(z) or softmax(z) over all experts; optionally the
//                       experts form n_groups equal groups of neighbours, a group scores the sum of its two largest s or its largest s, and
//                       only experts of the keep_groups best groups can be chosen; the `top` largest s among those are chosen (ties: the
//                       lower index); their weights are the scores themselves, or the scores over their sum
//   moe_combine_kernel  x <- x + sum of a token's `top` expert rows with their weights, in slot order
//   moe_sort_kernel     the step's (token, slot) pairs ordered by expert, cut into row tiles of one expert each
//   moe_gemm_kernel     out[pair] = A[row of pair] . W_expert(pair)^T in IEEE fp32 for every tile, with the row products' fused epilogues
//                       (gated activation on interleaved gate | up columns, plain store)
//
// The weighted sum over a token's chosen experts is left to the consumer (group_norm_residual_kernel sums the `top` rows in slot order),
// so no float atomics are needed and results do not depend on how the pairs were ordered.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "mix_ops.cuh"

namespace xalm {
namespace mix {

struct MoeRouteArgs {
	const float* h; // (T, K)
	int ldh;
	const void* w;  // (E, K) bf16 or fp32
	int w_bf16;
	int E, top, K;
	int n_groups, keep_groups; // n_groups <= 1: every expert can be chosen
	int* idx;   // (T, top)
	float* wgt; // (T, top)
	const SeqStep* step;
	int score_kind;  // MOE_SCORE_SIGMOID (0) or MOE_SCORE_SOFTMAX: exp(z - max z) / sum over all experts
	int group_kind;  // MOE_GROUP_TOP2_SUM (0) or MOE_GROUP_MAX: what a group scores
	int renormalise; // 1: the chosen weights are divided by (their sum + renorm_eps)
	float renorm_eps;
};
enum { MOE_SCORE_SIGMOID = 0, MOE_SCORE_SOFTMAX = 1 };
enum { MOE_GROUP_TOP2_SUM = 0, MOE_GROUP_MAX = 1 };

// (value, index) argmax over a warp; ties go to the lower index; index -1 = nothing
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
	for (int s = 16; s >= 1; s >>= 1) {
		const float ov = __shfl_xor_sync(0xffffffffu, v, s);
		const int oi = __shfl_xor_sync(0xffffffffu, i, s);
		if (oi >= 0 && (i < 0 || ov > v || (ov == v && oi < i))) { v = ov; i = oi; }
	}
}

template <typename WT>
__global__ void __launch_bounds__(256) moe_router_kernel(MoeRouteArgs a) {
	extern __shared__ float sm[];
	float* hs = sm;                      // K
	float* sc = hs + a.K;                // E scores
	float* gsc = sc + a.E;               // n_groups
	int* flag = reinterpret_cast<int*>(gsc + max(a.n_groups, 1)); // E: 1 = may be chosen, 0 = not (or already chosen)
	const int t = blockIdx.x, tid = threadIdx.x, nth = blockDim.x, lane = tid & 31, warp = tid >> 5, nw = nth >> 5;
	if (t >= a.step->n) return;
	for (int k = tid; k < a.K; k += nth) hs[k] = a.h[(size_t) t * a.ldh + k];
	__syncthreads();
	const WT* W = reinterpret_cast<const WT*>(a.w);
	for (int e = warp; e < a.E; e += nw) {
		float z = 0.f;
		if ((a.K & 7) == 0 && (reinterpret_cast<uintptr_t>(a.w) & 31) == 0) {
#pragma unroll 4
			for (int k = lane * 8; k < a.K; k += 256) {
				float wv[8];
				ld8(W + (size_t) e * a.K + k, wv);
#pragma unroll
				for (int i = 0; i < 8; i++) z = fmaf(wv[i], hs[k + i], z);
			}
		} else
			for (int k = lane; k < a.K; k += 32) z = fmaf(ldf(W + (size_t) e * a.K + k), hs[k], z);
		z = warp_sum(z);
		if (lane == 0) sc[e] = a.score_kind == MOE_SCORE_SOFTMAX ? z : sigmoidf_(z);
	}
	__syncthreads();
	if (warp != 0) return;
	if (a.score_kind == MOE_SCORE_SOFTMAX) {
		float zm = -INFINITY, den = 0.f;
		for (int e = lane; e < a.E; e += 32) zm = fmaxf(zm, sc[e]);
		zm = warp_max(zm);
		for (int e = lane; e < a.E; e += 32) den += expf(sc[e] - zm);
		den = warp_sum(den);
		for (int e = lane; e < a.E; e += 32) sc[e] = expf(sc[e] - zm) / den;
		__syncwarp();
	}
	const int ng = a.n_groups > 1 ? a.n_groups : 1, gsz = a.E / ng;
	if (ng > 1) {
		for (int g = lane; g < ng; g += 32) { // sum of the group's two largest scores
			float m1 = -INFINITY, m2 = -INFINITY;
			for (int j = 0; j < gsz; j++) {
				const float v = sc[g * gsz + j];
				if (v > m1) { m2 = m1; m1 = v; }
				else if (v > m2) m2 = v;
			}
			gsc[g] = (gsz > 1 && a.group_kind == MOE_GROUP_TOP2_SUM) ? m1 + m2 : m1;
		}
		for (int e = lane; e < a.E; e += 32) flag[e] = 0;
		__syncwarp();
		for (int r = 0; r < a.keep_groups; r++) {
			float bv = -INFINITY;
			int bi = -1;
			for (int g = lane; g < ng; g += 32)
				if (gsc[g] != -INFINITY && (bi < 0 || gsc[g] > bv)) { bv = gsc[g]; bi = g; }
			warp_argmax(bv, bi);
			if (bi < 0) break;
			for (int j = lane; j < gsz; j += 32) flag[bi * gsz + j] = 1;
			if (lane == 0) gsc[bi] = -INFINITY;
			__syncwarp();
		}
	} else {
		for (int e = lane; e < a.E; e += 32) flag[e] = 1;
		__syncwarp();
	}
	for (int r = 0; r < a.top; r++) {
		float bv = -INFINITY;
		int bi = -1;
		for (int e = lane; e < a.E; e += 32)
			if (flag[e] && (bi < 0 || sc[e] > bv)) { bv = sc[e]; bi = e; }
		warp_argmax(bv, bi);
		if (lane == 0) {
			a.idx[(size_t) t * a.top + r] = bi < 0 ? 0 : bi;
			a.wgt[(size_t) t * a.top + r] = bi < 0 ? 0.f : bv;
			if (bi >= 0) flag[bi] = 0;
		}
		__syncwarp();
	}
	if (a.renormalise) {
		float tot = 0.f;
		for (int r = lane; r < a.top; r += 32) tot += a.wgt[(size_t) t * a.top + r]; // written by lane 0 above
		tot = warp_sum(tot) + a.renorm_eps;
		for (int r = lane; r < a.top; r += 32) a.wgt[(size_t) t * a.top + r] /= tot;
	}
}

// ---- x <- x + sum_p w[t, p] y[row(t, p)]: the chosen experts' rows of a token joined in slot order (a fixed order: the same bits every run) ----
struct MoeCombineArgs {
	const float* y;      // (rows * top, ldy)
	int ldy, top, width;
	const float* wgt;    // (rows, top)
	const int* part_row; // (rows, top) row of y that holds slot p of token t, or NULL: t * top + p
	const float* x_in;   // (rows, width) or NULL
	float* x_out;        // (rows, width); may be x_in
	const SeqStep* step;
};
// grid (tokens, column parts): a one-token step spreads its row over several CTAs
static __global__ void moe_combine_kernel(MoeCombineArgs a) {
	const int t = blockIdx.x;
	if (t >= a.step->n) return;
	for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < a.width; c += gridDim.y * blockDim.x) {
		float v = 0.f;
		for (int p = 0; p < a.top; p++) {
			const size_t pk = (size_t) t * a.top + p;
			v = fmaf(a.wgt[pk], a.y[(a.part_row ? (size_t) a.part_row[pk] : pk) * a.ldy + c], v);
		}
		const size_t at = (size_t) t * a.width + c;
		a.x_out[at] = a.x_in ? a.x_in[at] + v : v;
	}
}
static inline int launch_moe_combine(const MoeCombineArgs& a, int rows, cudaStream_t s) {
	const int nt = norm_threads(a.width), parts = rows >= 64 ? 1 : std::min(16, (a.width + nt - 1) / nt);
	moe_combine_kernel<<<dim3(rows, parts), nt, 0, s>>>(a);
	return launch_check("moe_combine");
}

constexpr int MOE_TM = 64; // rows of a tile

struct MoeSortArgs {
	const int* idx; // (T, top)
	int top, E;
	const SeqStep* step;
	int* sorted;  // (T * top) pair ids, expert after expert
	int* tiles;   // (max_tiles, 3): expert, first place in `sorted`, rows
	int* n_tiles; // (1)
	int* off;     // (E + 1) first place of every expert in `sorted`, or NULL
	int* inv;     // (T * top) place of every pair in `sorted`, or NULL
};
// one CTA; shared memory: 2 E + 1 ints
static __global__ void moe_sort_kernel(MoeSortArgs a) {
	extern __shared__ int smi[];
	int* cnt = smi;           // E
	int* off = smi + a.E;     // E + 1
	const int tid = threadIdx.x, nth = blockDim.x, P = a.step->n * a.top;
	for (int e = tid; e < a.E; e += nth) cnt[e] = 0;
	__syncthreads();
	for (int p = tid; p < P; p += nth) atomicAdd(&cnt[a.idx[p]], 1);
	__syncthreads();
	if (tid == 0) {
		int at = 0, nt = 0;
		for (int e = 0; e < a.E; e++) {
			off[e] = at;
			for (int r = 0; r < cnt[e]; r += MOE_TM) {
				a.tiles[3 * nt] = e;
				a.tiles[3 * nt + 1] = at + r;
				a.tiles[3 * nt + 2] = min(MOE_TM, cnt[e] - r);
				nt++;
			}
			at += cnt[e];
		}
		off[a.E] = at;
		*a.n_tiles = nt;
	}
	__syncthreads();
	for (int e = tid; e < a.E; e += nth) cnt[e] = off[e]; // cursors
	__syncthreads();
	for (int p = tid; p < P; p += nth) { // the order inside an expert does not matter: rows are independent
		const int place = atomicAdd(&cnt[a.idx[p]], 1);
		a.sorted[place] = p;
		if (a.inv) a.inv[p] = place;
	}
	if (a.off)
		for (int e = tid; e <= a.E; e += nth) a.off[e] = off[e];
}

// rows of the pairs in sorted order, one after the other: dst[place] = src[sorted[place] / div] (the tensor-core products want each expert's rows
// contiguous)
static __global__ void moe_gather_kernel(const float* __restrict__ src, int lds, int div, const int* __restrict__ sorted, const SeqStep* step, int top, int width,
                                         float* __restrict__ dst) {
	const int place = blockIdx.x;
	if (place >= step->n * top) return;
	const float* row = src + (size_t) (sorted[place] / div) * lds;
	for (int c = threadIdx.x; c < width; c += blockDim.x) dst[(size_t) place * width + c] = row[c];
}

struct MoeGemmArgs {
	const float* A; // rows of lda floats; pair p reads row p / a_div
	int lda, a_div;
	const void* W;  // (E, N, K) bf16 or fp32
	int N, K;
	const int* sorted;
	const int* tiles;
	const int* n_tiles;
	RowsEpi e;      // rows of the output are pair ids
	// steps of a few tokens skip the tile list: one matvec per (token, slot) pair
	const int* idx; // (T, top) the pairs' experts
	const SeqStep* step;
	int top;
};

// 64 x 64 x 16 tiles, 4 x 4 per thread, as rows_gemm_kernel; blockIdx.y walks the tile list
template <typename WT>
__global__ void __launch_bounds__(256) moe_gemm_kernel(MoeGemmArgs a) {
	constexpr int BM = MOE_TM, BN = 64, BK = 16;
	__shared__ float As[BK][BM + 4];
	__shared__ float Ws[BK][BN + 4];
	__shared__ int prow[BM];
	if ((int) blockIdx.y >= *a.n_tiles) return;
	const int ex = a.tiles[3 * blockIdx.y], first = a.tiles[3 * blockIdx.y + 1], rows = a.tiles[3 * blockIdx.y + 2];
	const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4, n0 = blockIdx.x * BN, N = a.N, K = a.K;
	const WT* W = reinterpret_cast<const WT*>(a.W) + (size_t) ex * N * K;
	if (tid < BM) prow[tid] = tid < rows ? a.sorted[first + tid] : -1;
	__syncthreads();
	float acc[4][4] = {};
	for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
		for (int i = 0; i < 4; i++) {
			const int idx = tid + i * 256, r = idx >> 4, k = idx & 15, gn = n0 + r, gk = k0 + k;
			const int pr = prow[r];
			As[k][r] = (pr >= 0 && gk < K) ? a.A[(size_t) (pr / a.a_div) * a.lda + gk] : 0.f;
			Ws[k][r] = (gn < N && gk < K) ? ldf(W + (size_t) gn * K + gk) : 0.f;
		}
		__syncthreads();
#pragma unroll
		for (int k = 0; k < BK; k++) {
			const float4 av4 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
			const float4 bv4 = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
			const float av[4] = {av4.x, av4.y, av4.z, av4.w}, bv[4] = {bv4.x, bv4.y, bv4.z, bv4.w};
#pragma unroll
			for (int i = 0; i < 4; i++)
#pragma unroll
				for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
		}
		__syncthreads();
	}
#pragma unroll
	for (int i = 0; i < 4; i++) {
		const int row = prow[ty * 4 + i];
		if (row < 0) continue;
		if (a.e.kind == EPI_GLU) {
#pragma unroll
			for (int j = 0; j < 4; j += 2) {
				const int col = n0 + tx * 4 + j;
				if (col + 1 < N) epi_apply(a.e, row, col, N, acc[i][j], acc[i][j + 1]);
			}
		} else {
#pragma unroll
			for (int j = 0; j < 4; j++) {
				const int col = n0 + tx * 4 + j;
				if (col < N) epi_apply(a.e, row, col, N, acc[i][j], 0.f);
			}
		}
	}
}

// ---- the same for steps of a few tokens: every (token, slot) pair is a matvec of its own expert (blockIdx.y = pair), a warp per pair of
// output columns, or KS warps of the CTA per pair of columns (each a slice of K) when there are too few columns to fill the machine ------
template <typename WT, int KS>
__global__ void __launch_bounds__(256) moe_matvec_kernel(MoeGemmArgs a) {
	__shared__ float red[8][2];
	const int p = blockIdx.y;
	if (p >= a.step->n * a.top) return;
	const int N = a.N, K = a.K;
	const WT* W = reinterpret_cast<const WT*>(a.W) + (size_t) a.idx[p] * N * K;
	const float* A = a.A + (size_t) (p / a.a_div) * a.lda;
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, ks = warp % KS;
	const int c0 = (blockIdx.x * (8 / KS) + warp / KS) * 2;
	const bool live = c0 < N, two = c0 + 1 < N;
	float acc0 = 0.f, acc1 = 0.f;
	if (live) {
		const WT* w0 = W + (size_t) c0 * K;
		const WT* w1 = W + (size_t) (two ? c0 + 1 : c0) * K;
		const bool vec = (K % 8 == 0) && (a.lda % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.W) & 31) == 0) && ((reinterpret_cast<uintptr_t>(a.A) & 15) == 0);
		if (vec) {
#pragma unroll 2
			for (int k = (ks * 32 + lane) * 8; k < K; k += 256 * KS) {
				float a0[8], a1[8], x[8];
				ld8(w0 + k, a0);
				ld8(w1 + k, a1);
				ld8(A + k, x);
#pragma unroll
				for (int i = 0; i < 8; i++) {
					acc0 = fmaf(a0[i], x[i], acc0);
					acc1 = fmaf(a1[i], x[i], acc1);
				}
			}
		} else {
			for (int k = ks * 32 + lane; k < K; k += 32 * KS) {
				const float x = A[k];
				acc0 = fmaf(ldf(w0 + k), x, acc0);
				acc1 = fmaf(ldf(w1 + k), x, acc1);
			}
		}
		acc0 = warp_sum(acc0);
		acc1 = warp_sum(acc1);
	}
	if (KS > 1) {
		if (lane == 0) { red[warp][0] = acc0; red[warp][1] = acc1; }
		__syncthreads();
		if (ks == 0 && lane == 0)
			for (int j = 1; j < KS; j++) { acc0 += red[warp + j][0]; acc1 += red[warp + j][1]; }
	}
	if (live && ks == 0 && lane == 0) {
		if (a.e.kind == EPI_GLU) {
			if (two) epi_apply(a.e, p, c0, N, acc0, acc1);
		} else {
			epi_apply(a.e, p, c0, N, acc0, 0.f);
			if (two) epi_apply(a.e, p, c0 + 1, N, acc1, 0.f);
		}
	}
}

// ---- launchers ------------------------------------------------------------------------------------------------------------------
static inline size_t moe_router_smem(int K, int E, int n_groups) { return (size_t) (K + 2 * E + std::max(n_groups, 1)) * 4; }
static inline int moe_prepare(int K, int E, int n_groups) { // outside a stream capture
	if (moe_router_smem(K, E, n_groups) > 48 * 1024) {
		XALM_CUDA_CHECK(cudaFuncSetAttribute(moe_router_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
		XALM_CUDA_CHECK(cudaFuncSetAttribute(moe_router_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
	}
	return XALM_OK;
}
static inline int moe_max_tiles(int pairs, int E) { return (pairs + MOE_TM - 1) / MOE_TM + E; }
static inline int launch_moe_router(const MoeRouteArgs& a, int rows, cudaStream_t s) {
	if (a.E <= 0 || a.top <= 0 || a.top > a.E) return set_error(XALM_ERR_INVALID, "router: %d of %d experts", a.top, a.E);
	if (a.n_groups > 1 && (a.E % a.n_groups || a.keep_groups <= 0 || a.keep_groups > a.n_groups || a.keep_groups * (a.E / a.n_groups) < a.top))
		return set_error(XALM_ERR_INVALID, "router: %d groups, %d kept, cannot hold %d of %d experts", a.n_groups, a.keep_groups, a.top, a.E);
	const size_t smem = moe_router_smem(a.K, a.E, a.n_groups);
	if (a.w_bf16) moe_router_kernel<__nv_bfloat16><<<rows, 256, smem, s>>>(a);
	else moe_router_kernel<float><<<rows, 256, smem, s>>>(a);
	return launch_check("moe_router");
}
static inline int launch_moe_sort(const MoeSortArgs& a, cudaStream_t s) {
	moe_sort_kernel<<<1, 1024, (size_t) (2 * a.E + 1) * 4, s>>>(a);
	return launch_check("moe_sort");
}
// pairs: host-side bound of the step's (token, slot) pairs
constexpr int MOE_MATVEC_PAIRS = 32; // up to this many pairs in a step, each pair is a matvec of its own
static inline int launch_moe_gemm(const MoeGemmArgs& a, bool w_bf16, int pairs, int E, cudaStream_t s) {
	if (pairs <= MOE_MATVEC_PAIRS && a.idx && a.step) {
		const int cols = (a.N + 1) / 2;
		int ks = 1; // warps per column pair: enough CTAs for two per SM, each slice of K at least 256 long
		while (ks < 8 && (long long) ((cols * ks + 7) / 8) * pairs < 296 && a.K >= 512 * ks) ks *= 2;
		const dim3 grid((cols * ks + 7) / 8, pairs);
#define XALM_MOE_MATVEC(WT_)                                                             \
	do {                                                                                 \
		if (ks == 1) moe_matvec_kernel<WT_, 1><<<grid, 256, 0, s>>>(a);                  \
		else if (ks == 2) moe_matvec_kernel<WT_, 2><<<grid, 256, 0, s>>>(a);             \
		else if (ks == 4) moe_matvec_kernel<WT_, 4><<<grid, 256, 0, s>>>(a);             \
		else moe_matvec_kernel<WT_, 8><<<grid, 256, 0, s>>>(a);                          \
	} while (0)
		if (w_bf16) XALM_MOE_MATVEC(__nv_bfloat16);
		else XALM_MOE_MATVEC(float);
#undef XALM_MOE_MATVEC
		return launch_check("moe_matvec");
	}
	const dim3 grid((a.N + 63) / 64, moe_max_tiles(pairs, E));
	if (w_bf16) moe_gemm_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(a);
	else moe_gemm_kernel<float><<<grid, 256, 0, s>>>(a);
	return launch_check("moe_gemm");
}

} // namespace mix
} // namespace xalm
