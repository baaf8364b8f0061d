// delta_ops.cuh — the gated delta rule as a token mixer, with the short causal convolutions in front of it:
//
//   delta_prep_kernel   per token: depthwise causal convolution over time (taps inputs per channel, the last column of the weight is
//                       the current token's, zeros before the sequence's start) + silu on the q | k | v channels; q and k heads to unit
//                       length (x / sqrt(sum x^2 + unit_eps), q also times q_scale); write strength beta = sigmoid(.) and decay
//                       g = exp(-exp(A_log) * softplus(. + dt_bias)) per head
//   delta_rule_kernel   per head, token after token:  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q   (the read-out sees the
//                       token's own write), then o / rms(o) * norm_w * silu(gate).  S (d x dv, fp32) is the sequence's recurrent state
//                       and stays in device memory between steps, as do the last taps - 1 inputs of every convolved channel.
//
// A column of S evolves on its own (u_c needs only S[:, c]): one to four neighbouring lanes own a column, its d values in their registers
// (d <= 256; beyond that in shared memory), k and q of the token are broadcast from shared memory, and the only sums across lanes are
// the two dot products inside a column's lanes and the per-head norm.
// The scan is sequential in the tokens by construction: the state keeps the exact fp32 recurrence.  Everything is fp32 (expf, log1pf).
#pragma once
#include <cuda_runtime.h>
#include <math.h>

#include "common.cuh"
#include "mix_ops.cuh"

namespace xalm {
namespace mix {

struct DeltaArgs {
	const float* proj; // (T, ld) raw projections of the step's tokens
	int ld;
	int q_off, k_off, v_off; // convolved channels: q (G * d), k (G * d), v (H * dv)
	int g_off, b_off, a_off; // output gate (H * dv), write strength (H), decay input (H)
	int H, G, d, dv, taps;
	const float *wq, *wk, *wv; // (channels, taps)
	const float *A_log, *dt_bias; // (H)
	const float* norm_w;       // (dv) or NULL
	float eps, unit_eps, q_scale;
	float* conv_state; // (taps - 1, 2 G d + H dv): the inputs of the last taps - 1 positions, oldest first
	float* state;      // (H, d, dv)
	float* prep;       // (T, ldp): q | k | v after convolution, silu and unit length, then beta (H), g (H)
	int ldp;
	float* out;        // (T, H * dv)
	const SeqStep* step;
};


// grid (tokens, 2 G + H): a CTA convolves one head — a q head, a k head (both scaled to unit length afterwards) or a v head; the CTA of
// the first head also computes the token's write strengths and decays
static __global__ void delta_prep_kernel(DeltaArgs a) {
	__shared__ float red[33];
	const int t = blockIdx.x, unit = blockIdx.y, tid = threadIdx.x, nth = blockDim.x;
	if (t >= a.step->n) return;
	const int nq = a.G * a.d, nv = a.H * a.dv, Cc = 2 * nq + nv, taps = a.taps;
	const int sec = unit < a.G ? 0 : unit < 2 * a.G ? 1 : 2;           // q, k, v
	const int n = sec == 2 ? a.dv : a.d;                               // channels of this head
	const int lc0 = sec == 0 ? unit * a.d : sec == 1 ? (unit - a.G) * a.d : (unit - 2 * a.G) * a.dv; // first channel inside its section
	const int cc0 = (sec == 0 ? 0 : sec == 1 ? nq : 2 * nq) + lc0;     // ... and among all convolved channels
	const int off = (sec == 0 ? a.q_off : sec == 1 ? a.k_off : a.v_off) + lc0;
	const float* wbase = (sec == 0 ? a.wq : sec == 1 ? a.wk : a.wv) + (size_t) lc0 * taps;
	float* prow = a.prep + (size_t) t * a.ldp;
	float ss = 0.f;
	// a thread's channels: c = tid + k * nth.  The first eight stay in registers for the scaling sweep; a head beyond 8 * nth channels parks
	// the rest unscaled in the output row and rescales them there.
	auto conv = [&](int c) {
		const float* w = wbase + (size_t) c * taps;
		float y = 0.f;
		for (int tau = 0; tau < taps; tau++) {
			const int r = t - (taps - 1) + tau; // row of this step, or (negative) one of the positions before it
			const float x = r >= 0 ? a.proj[(size_t) r * a.ld + off + c] : a.conv_state[(size_t) (taps - 1 + r) * Cc + cc0 + c];
			y = fmaf(w[tau], x, y);
		}
		return y * sigmoidf_(y);
	};
	float keep[8];
#pragma unroll
	for (int k = 0; k < 8; k++) {
		const int c = tid + k * nth;
		keep[k] = c < n ? conv(c) : 0.f;
		ss = fmaf(keep[k], keep[k], ss);
	}
	for (int c = tid + 8 * nth; c < n; c += nth) {
		const float y = conv(c);
		prow[cc0 + c] = y;
		ss = fmaf(y, y, ss);
	}
	float r = 1.f;
	if (sec != 2) r = (sec == 0 ? a.q_scale : 1.f) / sqrtf(block_sum(ss, red) + a.unit_eps);
#pragma unroll
	for (int k = 0; k < 8; k++) {
		const int c = tid + k * nth;
		if (c < n) prow[cc0 + c] = keep[k] * r;
	}
	if (sec != 2)
		for (int c = tid + 8 * nth; c < n; c += nth) prow[cc0 + c] *= r;
	if (unit == 0)
		for (int h = tid; h < a.H; h += nth) {
			const float* row = a.proj + (size_t) t * a.ld;
			prow[Cc + h] = sigmoidf_(row[a.b_off + h]);
			prow[Cc + a.H + h] = expf(-expf(a.A_log[h]) * softplusf_(row[a.a_off + h] + a.dt_bias[h]));
		}
}

constexpr int DELTA_TT = 16; // tokens staged at a time

// A column of the state is shared by NS neighbouring lanes, each keeping DS of its d values in registers (d <= DS * NS); the two dot
// products of a token are completed with log2(NS) shuffles.  DS == 0: one thread per column, the state in shared memory (any d that fits).
// one 4-byte element, global -> shared, without a register in between: every copy of a tile is in flight at once
__device__ __forceinline__ void delta_cp4(float* dst, const float* src) {
	asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned) __cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <int DS, int NS>
__global__ void __launch_bounds__(512) delta_rule_kernel(DeltaArgs a) {
	extern __shared__ __align__(16) float sm[];
	const int h = blockIdx.x, tid = threadIdx.x, nth = blockDim.x, lane = tid & 31, warp = tid >> 5, nw = nth >> 5;
	const int d = a.d, dv = a.dv, dp = DS > 0 ? DS * NS : ((d + 3) & ~3), hk = h / (a.H / a.G);
	const int nq = a.G * d, Cc = 2 * nq + a.H * dv;
	// a token's k (and q) in shared memory: the NS slices 4 floats apart from one another's end, so that the 16-byte reads of a warp's NS
	// slices fall on different banks
	const int dps = DS > 0 ? NS * (DS + 4) : dp;
	// two tile buffers (the next tile's copies fly while this one is scanned): k | q | v | gate | beta, g
	const int tile_floats = DELTA_TT * (2 * dps + 2 * dv + 2);
	float* och = sm + 2 * tile_floats;      // TT * dv
	float* Ssh = och + DELTA_TT * dv;       // DS == 0: dp * nth
	const int T = a.step->n;
	const int c = tid / NS, sl = tid % NS, i0 = sl * DS; // this thread's column and its slice of d
	const bool live = c < dv;
	float* st = a.state + (size_t) h * d * dv;
	float S[DS > 0 ? DS : 1];
	if constexpr (DS > 0) {
#pragma unroll
		for (int i = 0; i < DS; i++) S[i] = (live && i0 + i < d) ? st[(size_t) (i0 + i) * dv + c] : 0.f;
	} else {
		for (int i = 0; i < dp; i++) Ssh[(size_t) i * nth + tid] = (live && i < d) ? st[(size_t) i * dv + c] : 0.f;
	}
	if (dp != d) { // channels beyond d that the scan reads stay zero: copies touch real channels only
		for (int x = tid; x < 2 * tile_floats; x += nth) sm[x] = 0.f;
		__syncthreads();
	}
	auto stage = [&](float* buf, int t0) {
		const int nt = min(DELTA_TT, T - t0);
		float *ks = buf, *qs = ks + DELTA_TT * dps, *vs = qs + DELTA_TT * dps, *gs = vs + DELTA_TT * dv, *bg = gs + DELTA_TT * dv;
		for (int x = tid; x < nt * d; x += nth) {
			const int tt = x / d, i = x % d;
			const float* prow = a.prep + (size_t) (t0 + tt) * a.ldp;
			const int at = tt * dps + (DS > 0 ? (i / (DS > 0 ? DS : 1)) * (DS + 4) + i % (DS > 0 ? DS : 1) : i);
			delta_cp4(ks + at, prow + nq + hk * d + i);
			delta_cp4(qs + at, prow + hk * d + i);
		}
		for (int x = tid; x < nt * dv; x += nth) {
			const int tt = x / dv, cc = x % dv;
			delta_cp4(vs + x, a.prep + (size_t) (t0 + tt) * a.ldp + 2 * nq + h * dv + cc);
			delta_cp4(gs + x, a.proj + (size_t) (t0 + tt) * a.ld + a.g_off + h * dv + cc);
		}
		for (int x = tid; x < nt * 2; x += nth) delta_cp4(bg + x, a.prep + (size_t) (t0 + (x >> 1)) * a.ldp + Cc + (x & 1) * a.H + h);
		asm volatile("cp.async.commit_group;" ::: "memory");
	};
	if (T > 0) stage(sm, 0);
	int cur = 0;
	for (int t0 = 0; t0 < T; t0 += DELTA_TT, cur ^= 1) {
		const int nt = min(DELTA_TT, T - t0);
		const float *ks = sm + cur * tile_floats, *qs = ks + DELTA_TT * dps, *vs = qs + DELTA_TT * dps, *gs = vs + DELTA_TT * dv, *bg = gs + DELTA_TT * dv;
		__syncthreads(); // the other buffer's last readers (the tile before this one) are done
		if (t0 + DELTA_TT < T) {
			stage(sm + (cur ^ 1) * tile_floats, t0 + DELTA_TT);
			asm volatile("cp.async.wait_group 1;" ::: "memory");
		} else asm volatile("cp.async.wait_group 0;" ::: "memory");
		__syncthreads();
		for (int tt = 0; tt < nt; tt++) { // every lane takes part (the shuffles want whole warps); dead columns compute on zeros
			const float beta = bg[2 * tt], g = bg[2 * tt + 1], v = live ? vs[tt * dv + c] : 0.f;
			float o;
			if constexpr (DS > 0) {
				const float4* k4 = reinterpret_cast<const float4*>(ks + tt * dps + sl * (DS + 4));
				const float4* q4 = reinterpret_cast<const float4*>(qs + tt * dps + sl * (DS + 4));
				float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
				for (int i = 0; i < DS; i += 4) {
					const float4 kk = k4[i >> 2];
					S[i] *= g; S[i + 1] *= g; S[i + 2] *= g; S[i + 3] *= g;
					d0 = fmaf(kk.x, S[i], d0); d1 = fmaf(kk.y, S[i + 1], d1); d2 = fmaf(kk.z, S[i + 2], d2); d3 = fmaf(kk.w, S[i + 3], d3);
				}
				float dk = (d0 + d1) + (d2 + d3);
#pragma unroll
				for (int s = 1; s < NS; s <<= 1) dk += __shfl_xor_sync(0xffffffffu, dk, s);
				const float u = beta * (v - dk);
				float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
				for (int i = 0; i < DS; i += 4) {
					const float4 kk = k4[i >> 2], qq = q4[i >> 2];
					S[i] = fmaf(kk.x, u, S[i]); S[i + 1] = fmaf(kk.y, u, S[i + 1]); S[i + 2] = fmaf(kk.z, u, S[i + 2]); S[i + 3] = fmaf(kk.w, u, S[i + 3]);
					o0 = fmaf(qq.x, S[i], o0); o1 = fmaf(qq.y, S[i + 1], o1); o2 = fmaf(qq.z, S[i + 2], o2); o3 = fmaf(qq.w, S[i + 3], o3);
				}
				o = (o0 + o1) + (o2 + o3);
#pragma unroll
				for (int s = 1; s < NS; s <<= 1) o += __shfl_xor_sync(0xffffffffu, o, s);
			} else {
				float d0 = 0.f, d1 = 0.f;
				for (int i = 0; i < dp; i += 2) {
					const float s0 = Ssh[(size_t) i * nth + tid] * g, s1 = Ssh[(size_t) (i + 1) * nth + tid] * g;
					Ssh[(size_t) i * nth + tid] = s0;
					Ssh[(size_t) (i + 1) * nth + tid] = s1;
					d0 = fmaf(ks[tt * dp + i], s0, d0);
					d1 = fmaf(ks[tt * dp + i + 1], s1, d1);
				}
				const float u = beta * (v - (d0 + d1));
				float o0 = 0.f, o1 = 0.f;
				for (int i = 0; i < dp; i += 2) {
					const float s0 = fmaf(ks[tt * dp + i], u, Ssh[(size_t) i * nth + tid]), s1 = fmaf(ks[tt * dp + i + 1], u, Ssh[(size_t) (i + 1) * nth + tid]);
					Ssh[(size_t) i * nth + tid] = s0;
					Ssh[(size_t) (i + 1) * nth + tid] = s1;
					o0 = fmaf(qs[tt * dp + i], s0, o0);
					o1 = fmaf(qs[tt * dp + i + 1], s1, o1);
				}
				o = o0 + o1;
			}
			if (live && sl == 0) och[tt * dv + c] = o;
		}
		__syncthreads();
		for (int tt = warp; tt < nt; tt += nw) { // per-head norm over the value channels, weight, output gate
			float r = 1.f;
			if (a.norm_w) {
				float ss = 0.f;
				for (int cc = lane; cc < dv; cc += 32) ss = fmaf(och[tt * dv + cc], och[tt * dv + cc], ss);
				ss = warp_sum(ss);
				r = 1.f / sqrtf(ss / (float) dv + a.eps);
			}
			float* orow = a.out + (size_t) (t0 + tt) * (a.H * dv) + h * dv;
			for (int cc = lane; cc < dv; cc += 32) {
				const float z = gs[tt * dv + cc];
				orow[cc] = och[tt * dv + cc] * r * (a.norm_w ? a.norm_w[cc] : 1.f) * (z * sigmoidf_(z));
			}
		}
	}
	if (live) {
		if constexpr (DS > 0) {
#pragma unroll
			for (int i = 0; i < DS; i++)
				if (i0 + i < d) st[(size_t) (i0 + i) * dv + c] = S[i];
		} else {
			for (int i = 0; i < d; i++) st[(size_t) i * dv + c] = Ssh[(size_t) i * nth + tid];
		}
	}
	// the inputs of the last taps - 1 positions become the convolution's state (delta_prep_kernel has read the old one: it ran before)
	const int keep = a.taps - 1;
	for (int cc = h * nth + tid; cc < Cc; cc += gridDim.x * nth) {
		const int sec = cc < nq ? 0 : cc < 2 * nq ? 1 : 2, lc = cc - (sec == 0 ? 0 : sec == 1 ? nq : 2 * nq);
		const int off = sec == 0 ? a.q_off : sec == 1 ? a.k_off : a.v_off;
		for (int r = 0; r < keep; r++) { // ascending: a row that is read has not been rewritten yet
			const int src = T - keep + r;
			a.conv_state[(size_t) r * Cc + cc] = src >= 0 ? a.proj[(size_t) src * a.ld + off + lc] : a.conv_state[(size_t) (r + T) * Cc + cc];
		}
	}
}

// How a head of d x dv is laid out: DS registers per thread and NS threads per column (DS 0: the shared-memory kernel, one thread per column)
struct DeltaShape {
	int DS, NS, threads;
};
static inline DeltaShape delta_shape(int d, int dv) {
	static const int opts[][2] = {{32, 1}, {32, 2}, {32, 4}, {64, 4}, {64, 2}, {64, 1}};
	for (const auto& o : opts)
		if (d <= o[0] * o[1] && dv * o[1] <= 512) return {o[0], o[1], (dv * o[1] + 31) / 32 * 32};
	return {0, 1, (dv + 31) / 32 * 32};
}
static inline size_t delta_rule_smem(int d, int dv) {
	const DeltaShape z = delta_shape(d, dv);
	const int dp = z.DS ? z.NS * (z.DS + 4) : ((d + 3) & ~3);
	return sizeof(float) * (2 * (size_t) DELTA_TT * (2 * dp + 2 * dv + 2) + (size_t) DELTA_TT * dv + (z.DS ? 0 : (size_t) dp * z.threads));
}
static inline bool delta_ok(int d, int dv) { return dv <= 512 && delta_rule_smem(d, dv) <= 200 * 1024; }
#define XALM_DELTA_DISPATCH(z_, CALL)                                      \
	do {                                                                   \
		if (z_.DS == 32 && z_.NS == 1) { CALL(32, 1); }                    \
		else if (z_.DS == 32 && z_.NS == 2) { CALL(32, 2); }               \
		else if (z_.DS == 32 && z_.NS == 4) { CALL(32, 4); }               \
		else if (z_.DS == 64 && z_.NS == 4) { CALL(64, 4); }               \
		else if (z_.DS == 64 && z_.NS == 2) { CALL(64, 2); }               \
		else if (z_.DS == 64 && z_.NS == 1) { CALL(64, 1); }               \
		else { CALL(0, 1); }                                               \
	} while (0)
static inline int delta_prepare(int d, int dv) { // outside a stream capture
	if (delta_rule_smem(d, dv) > 48 * 1024) {
		const DeltaShape z = delta_shape(d, dv);
#define XALM_DELTA_ATTR(DS_, NS_) XALM_CUDA_CHECK(cudaFuncSetAttribute(delta_rule_kernel<DS_, NS_>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024))
		XALM_DELTA_DISPATCH(z, XALM_DELTA_ATTR);
#undef XALM_DELTA_ATTR
	}
	return XALM_OK;
}
// rows: tokens of the step (host-side bound); two launches
static inline int launch_delta(const DeltaArgs& a, int rows, cudaStream_t s) {
	if (a.H % a.G || a.taps < 1 || !delta_ok(a.d, a.dv)) return set_error(XALM_ERR_UNSUPPORTED, "delta rule: heads %d / %d, state %d x %d", a.H, a.G, a.d, a.dv);
	delta_prep_kernel<<<dim3(rows, 2 * a.G + a.H), 128, 0, s>>>(a);
	XALM_TRY(launch_check("delta_prep"));
	const DeltaShape z = delta_shape(a.d, a.dv);
	const size_t smem = delta_rule_smem(a.d, a.dv);
#define XALM_DELTA_LAUNCH(DS_, NS_) delta_rule_kernel<DS_, NS_><<<a.H, z.threads, smem, s>>>(a)
	XALM_DELTA_DISPATCH(z, XALM_DELTA_LAUNCH);
#undef XALM_DELTA_LAUNCH
	return launch_check("delta_rule");
}

} // namespace mix
} // namespace xalm
