// conv_ops.cuh — short causal convolutions over time whose last inputs belong to the sequence, as mechanisms that another design can use:
//
//   norm_conv_kernel    what a sublayer reads: the grouped RMS norm of the residual row (the row split into `groups` equal consecutive
//                       parts, each over its own sqrt(mean(part^2) + eps), times a weight), then h <- h + conv(h) with a depthwise
//                       causal convolution of `taps` inputs per channel over the normed rows.  Up to two readers of the same residual
//                       (a token mixer and a feed-forward that run side by side) are served by one launch: blockIdx.y = reader.
//   short_conv_kernel   y[t, c] = act(bias[c] + sum_j w[c, j] x[t - taps + 1 + j, c]) on a run of channels of a row buffer (the last
//                       column of w is the current row's, zeros before the sequence's start)
//
// Both keep the inputs of the last taps - 1 positions in device memory ("hist", oldest first) between steps.  A CTA walks its rows in
// order; rows before its first one come from the step's earlier rows or from hist.  When ONE CTA (per reader / channel block) covers
// the whole step it rewrites hist itself at the end: every thread reads and writes only its own channels, so nothing races, and a
// one-token step needs no second launch.  When several CTAs share a step, the CTA that holds the step's last taps - 1 rows writes them
// to "stage" instead, and the launcher copies stage over hist behind the kernel (device to device): no CTA then writes what another reads.
// Everything is fp32.
#pragma once
#include <cuda_runtime.h>
#include <math.h>

#include "common.cuh"
#include "mix_ops.cuh"

namespace xalm {
namespace mix {

constexpr int CONV_MAX_TAPS = 8;
constexpr int NORM_CONV_ROWS = 8;   // rows per CTA of norm_conv_kernel (>= taps - 1)
constexpr int SHORT_CONV_ROWS = 16; // rows per CTA of short_conv_kernel (>= taps - 1)

struct NormConvArgs {
	const float* x; // (T, width) the residual rows
	int width, groups, taps, readers;
	float eps;
	const float* w[2];  // (width) norm weight of each reader
	const float* cw[2]; // (width, taps) convolution weight of each reader
	float* hist[2];     // (taps - 1, width) normed rows of the last positions
	float* stage[2];    // (taps - 1, width)
	float* out[2];      // (T, width)
	const SeqStep* step;
};

// grid (ceil(T / NORM_CONV_ROWS), readers, groups), 256 threads.  A CTA serves the channels of ONE norm group for rows [r0, r1) and needs the
// taps - 1 rows before them as well: a group's norm needs no other group's channels, so a one-token step spreads over groups x readers CTAs.
// Phase 1, the norms' sums: the CTA's warps are dealt over those rows (all eight on the one row of a one-token step, one per row in a
// long pass), each summing its share of the group's squares -> 1 / rms per row in shared memory.  Phase 2, per channel: a thread loads its
// channel's value of every row at once (independent loads), then walks the rows with the window of the last `taps` normed values in
// registers.  Nothing but the 1 / rms table lives in shared memory, so many CTAs fit an SM.
// TAPS: the convolution's length at compile time (short windows and row lists in few registers); 0: read from the arguments, up to CONV_MAX_TAPS + 1
constexpr int NORM_CONV_SPAN = NORM_CONV_ROWS + CONV_MAX_TAPS; // most rows a CTA touches
template <int TAPS>
__global__ void __launch_bounds__(256) norm_conv_kernel(NormConvArgs a) {
	extern __shared__ float sm[];
	constexpr int M = TAPS ? TAPS : CONV_MAX_TAPS + 1, SPAN = NORM_CONV_ROWS + M - 1;
	const int W = a.width, taps = TAPS ? TAPS : a.taps, keep = taps - 1, rd = blockIdx.y, gs = W / a.groups, c0 = blockIdx.z * gs;
	const int tid = threadIdx.x, nth = blockDim.x, lane = tid & 31, warp = tid >> 5, nw = nth >> 5;
	const int n = a.step->n, r0 = blockIdx.x * NORM_CONV_ROWS, r1 = min(n, r0 + NORM_CONV_ROWS);
	if (r0 >= n) return;
	const int e0 = r0 - keep, ef = max(e0, 0), rows = r1 - ef; // rows of this step the CTA norms: ef .. r1 - 1
	int wpr = 1;                                               // warps per row
	while (wpr * 2 * rows <= nw) wpr *= 2;
	float* rinv = sm;                                          // NORM_CONV_SPAN
	float* psum = sm + NORM_CONV_SPAN;                         // NORM_CONV_SPAN * wpr
	for (int ri = warp / wpr; ri < rows; ri += nw / wpr) {
		const int part = warp % wpr;
		const float* xr = a.x + (size_t) (ef + ri) * W + c0;
		float ss = 0.f;
#pragma unroll 4
		for (int c = part * 32 + lane; c < gs; c += wpr * 32) {
			const float v = xr[c];
			ss = fmaf(v, v, ss);
		}
		ss = warp_sum(ss);
		if (lane == 0) psum[ri * wpr + part] = ss;
	}
	__syncthreads();
	for (int ri = tid; ri < rows; ri += nth) {
		float ss = 0.f;
		for (int p = 0; p < wpr; p++) ss += psum[ri * wpr + p];
		rinv[ri] = 1.f / sqrtf(ss / (float) gs + a.eps);
	}
	__syncthreads();
	const float *w = a.w[rd], *cw = a.cw[rd];
	float *hist = a.hist[rd], *out = a.out[rd];
	for (int c = c0 + tid; c < c0 + gs; c += nth) {
		float v[SPAN], win[M], wr[M];
#pragma unroll
		for (int i = 0; i < SPAN; i++) {
			const int e = e0 + i;
			v[i] = e >= r1 ? 0.f : e < 0 ? hist[(size_t) (keep + e) * W + c] : a.x[(size_t) e * W + c];
		}
		const float wc = w[c];
#pragma unroll
		for (int j = 0; j < M; j++) {
			const int jj = j - (M - taps);
			wr[j] = jj >= 0 ? cw[(size_t) c * taps + jj] : 0.f;
			win[j] = 0.f;
		}
#pragma unroll
		for (int i = 0; i < SPAN; i++) {
			const int e = e0 + i;
			if (e < r1) {
				const float h = e < 0 ? v[i] : v[i] * rinv[e - ef] * wc;
#pragma unroll
				for (int j = 0; j < M - 1; j++) win[j] = win[j + 1];
				win[M - 1] = h;
				if (e >= r0) {
					float y = h;
#pragma unroll
					for (int j = 0; j < M; j++) y = fmaf(wr[j], win[j], y);
					out[(size_t) e * W + c] = y;
				}
				if (gridDim.x > 1 && e >= n - keep && e >= r0) a.stage[rd][(size_t) (e - (n - keep)) * W + c] = h;
			}
		}
		if (gridDim.x == 1)
#pragma unroll
			for (int j = 0; j < M; j++) {
				const int i = j - (M - keep);
				if (i >= 0) hist[(size_t) i * W + c] = win[j];
			}
	}
}
static inline size_t norm_conv_smem(int width, int taps, int groups) {
	(void) width; (void) taps; (void) groups;
	return (size_t) NORM_CONV_SPAN * (1 + 8) * 4;
}
static inline int norm_conv_prepare(int width, int taps, int groups) { // nothing to raise: the kernel's shared memory does not grow with the row
	if (groups <= 0 || width % groups || groups > 65535) return set_error(XALM_ERR_INVALID, "norm: %d groups do not divide a row of %d", groups, width);
	(void) taps;
	return XALM_OK;
}
// rows: the step's tokens.  One or two launches' worth of work on s: the kernel, then (steps of more than NORM_CONV_ROWS rows) the copy of the
// staged rows over hist; hist[0] .. hist[readers - 1] and stage[...] must each be one allocation of readers * (taps - 1) * width floats
static inline int launch_norm_conv(const NormConvArgs& a, int rows, cudaStream_t s, int* launches = nullptr) {
	if (a.groups <= 0 || a.width % a.groups) return set_error(XALM_ERR_INVALID, "norm: %d groups do not divide a row of %d", a.groups, a.width);
	if (a.taps < 1 || a.taps > CONV_MAX_TAPS + 1 || a.readers < 1 || a.readers > 2) return set_error(XALM_ERR_UNSUPPORTED, "norm + convolution: %d taps, %d readers", a.taps, a.readers);
	const int blocks = (rows + NORM_CONV_ROWS - 1) / NORM_CONV_ROWS;
	const int gs = a.width / a.groups, nt = gs >= 256 ? 256 : gs >= 128 ? 128 : 64;
	const dim3 grid(blocks, a.readers, a.groups);
	const size_t smem = norm_conv_smem(a.width, a.taps, a.groups);
	if (a.taps == 1) norm_conv_kernel<1><<<grid, nt, smem, s>>>(a);
	else if (a.taps == 2) norm_conv_kernel<2><<<grid, nt, smem, s>>>(a);
	else if (a.taps == 3) norm_conv_kernel<3><<<grid, nt, smem, s>>>(a);
	else if (a.taps == 4) norm_conv_kernel<4><<<grid, nt, smem, s>>>(a);
	else norm_conv_kernel<0><<<grid, nt, smem, s>>>(a);
	XALM_TRY(launch_check("norm_conv"));
	if (launches) *launches = 1;
	if (blocks > 1 && a.taps > 1) {
		XALM_CUDA_CHECK(cudaMemcpyAsync(a.hist[0], a.stage[0], (size_t) a.readers * (a.taps - 1) * a.width * 4, cudaMemcpyDeviceToDevice, s));
		if (launches) *launches = 2;
	}
	return XALM_OK;
}

struct ShortConvArgs {
	const float* in; // (T, ld_in): the convolved channels at columns in_off ..
	float* out;      // (T, ld_out): results at columns out_off .. (may be other columns of the same buffer)
	int ld_in, in_off, ld_out, out_off;
	int C, taps;
	const float* w;    // (C, taps)
	const float* bias; // (C) or NULL
	int act;           // ACT_NONE or ACT_SILU
	float* hist;       // (taps - 1, C) raw inputs of the last positions
	float* stage;      // (taps - 1, C)
	const SeqStep* step;
};

// grid (ceil(C / 128), ceil(T / SHORT_CONV_ROWS)), 128 threads: a thread per channel, the window of its last inputs in registers
static __global__ void short_conv_kernel(ShortConvArgs a) {
	const int c = blockIdx.x * blockDim.x + threadIdx.x, taps = a.taps, keep = taps - 1;
	const int n = a.step->n, r0 = blockIdx.y * SHORT_CONV_ROWS, r1 = min(n, r0 + SHORT_CONV_ROWS);
	if (c >= a.C || r0 >= n) return;
	float win[CONV_MAX_TAPS], wr[CONV_MAX_TAPS]; // right-aligned: the last entry is the current row's
#pragma unroll
	for (int j = 0; j < CONV_MAX_TAPS; j++) { // entry j holds row r0 - CONV_MAX_TAPS + j before row r0 is shifted in
		const int jj = j - (CONV_MAX_TAPS - taps), e = r0 - CONV_MAX_TAPS + j;
		wr[j] = jj >= 0 ? a.w[(size_t) c * taps + jj] : 0.f;
		win[j] = jj <= 0 ? 0.f : e < 0 ? a.hist[(size_t) (keep + e) * a.C + c] : a.in[(size_t) e * a.ld_in + a.in_off + c];
	}
	const float b = a.bias ? a.bias[c] : 0.f;
	for (int t = r0; t < r1; t++) {
#pragma unroll
		for (int j = 0; j < CONV_MAX_TAPS - 1; j++) win[j] = win[j + 1];
		win[CONV_MAX_TAPS - 1] = a.in[(size_t) t * a.ld_in + a.in_off + c];
		float y = b;
#pragma unroll
		for (int j = 0; j < CONV_MAX_TAPS; j++) y = fmaf(wr[j], win[j], y);
		a.out[(size_t) t * a.ld_out + a.out_off + c] = a.act == ACT_SILU ? y * sigmoidf_(y) : y;
		if (gridDim.y > 1 && t >= n - keep) a.stage[(size_t) (t - (n - keep)) * a.C + c] = win[CONV_MAX_TAPS - 1];
	}
	if (gridDim.y == 1)
#pragma unroll
		for (int j = 0; j < CONV_MAX_TAPS; j++) {
			const int i = j - (CONV_MAX_TAPS - keep);
			if (i >= 0) a.hist[(size_t) i * a.C + c] = win[j];
		}
}
static inline int launch_short_conv(const ShortConvArgs& a, int rows, cudaStream_t s, int* launches = nullptr) {
	if (a.taps < 1 || a.taps > CONV_MAX_TAPS) return set_error(XALM_ERR_UNSUPPORTED, "short convolution: %d taps (1 to %d)", a.taps, CONV_MAX_TAPS);
	const int blocks = (rows + SHORT_CONV_ROWS - 1) / SHORT_CONV_ROWS;
	short_conv_kernel<<<dim3((a.C + 127) / 128, blocks), 128, 0, s>>>(a);
	XALM_TRY(launch_check("short_conv"));
	if (launches) *launches = 1;
	if (blocks > 1 && a.taps > 1) {
		XALM_CUDA_CHECK(cudaMemcpyAsync(a.hist, a.stage, (size_t) (a.taps - 1) * a.C * 4, cudaMemcpyDeviceToDevice, s));
		if (launches) *launches = 2;
	}
	return XALM_OK;
}

} // namespace mix
} // namespace xalm
