// latent_ops.cuh — attention whose keys and values live in a low-rank latent, as mechanisms that another design can use on their own:
//
//   latent_post_kernel   after the stacked down projections [q latent | kv latent | shared rotated key] of a token: RMS norm (plain weight)
//                        of the query latent -> a compact buffer; RMS norm of the kv latent and the rotary turn of the shared key part ->
//                        the token's cache row [latent | rotated key] (fp32 or bf16).  The cache keeps nothing else of the token.
//   rope_heads_kernel    rotary positions on the first 2 * rot_half entries of a run of heads (rotate-half pairs, angle = position * freq[i]
//                        in fp32), from one buffer to another or in place; entries past the rotated ones are copied when the buffers differ
//
// The attention itself runs on the sliding-window kernels of mix_ops.cuh in their "absorbed" form: one shared key/value head whose key row
// is the cache row and whose value is the latent slice of the same row (SwaArgs.ldk / ldv), queries mapped into the latent by a batched
// per-head product with the transposed key expansion (rows products with RowsEpi.batch_*), and the value expansion as a second batched
// product on the attention's output.  score_h(i, j) = (W_uk,h^T q_h(i)) . c(j) + q_rot,h(i) . k_rot(j) equals q_h(i) . (W_uk,h c(j)) + ...
// up to fp32 rounding, and no per-head key or value is ever written to memory.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "mix_ops.cuh"

namespace xalm {
namespace mix {

struct LatentPostArgs {
	const float* proj; // (T, ld)
	int ld;
	int q_off, q_rank;   // the query latent's columns; q_rank 0: none
	const float* q_norm; // (q_rank) plain weight
	float* cq;           // (T, ldc) normed query latent
	int ldc;
	int kv_off, kv_rank, rot; // the kv latent's columns, followed by `rot` columns of the shared rotated key; kv_rank 0: this layer reads another's cache
	const float* kv_norm;     // (kv_rank)
	const float* freq;        // (rot / 2), NULL when rot == 0
	float eps;
	void* cache;              // (ring, kv_rank + rot)
	int cache_f32, ring;      // position p lives in row p % ring
	const SeqStep* step;
};

// one CTA per token; shared memory: 33 floats
static __global__ void latent_post_kernel(LatentPostArgs a) {
	__shared__ float red[33];
	const int t = blockIdx.x, tid = threadIdx.x, nth = blockDim.x;
	if (t >= a.step->n) return;
	const float* row = a.proj + (size_t) t * a.ld;
	const int pos = a.step->pos0 + t;
	if (a.q_rank) {
		float ss = 0.f;
		for (int c = tid; c < a.q_rank; c += nth) ss = fmaf(row[a.q_off + c], row[a.q_off + c], ss);
		const float r = 1.f / sqrtf(block_sum(ss, red) / (float) a.q_rank + a.eps);
		for (int c = tid; c < a.q_rank; c += nth) a.cq[(size_t) t * a.ldc + c] = row[a.q_off + c] * r * a.q_norm[c];
	}
	if (!a.kv_rank) return;
	float ss = 0.f;
	for (int c = tid; c < a.kv_rank; c += nth) ss = fmaf(row[a.kv_off + c], row[a.kv_off + c], ss);
	const float r = 1.f / sqrtf(block_sum(ss, red) / (float) a.kv_rank + a.eps);
	const size_t at = (size_t) (pos % a.ring) * (a.kv_rank + a.rot);
	for (int c = tid; c < a.kv_rank; c += nth) {
		const float v = row[a.kv_off + c] * r * a.kv_norm[c];
		if (a.cache_f32) ((float*) a.cache)[at + c] = v;
		else ((__nv_bfloat16*) a.cache)[at + c] = __float2bfloat16_rn(v);
	}
	const int half = a.rot / 2;
	for (int c = tid; c < half; c += nth) {
		float sn, cs;
		sincosf((float) pos * a.freq[c], &sn, &cs);
		const float u = row[a.kv_off + a.kv_rank + c], v = row[a.kv_off + a.kv_rank + c + half];
		const float x = u * cs - v * sn, y = v * cs + u * sn;
		if (a.cache_f32) {
			((float*) a.cache)[at + a.kv_rank + c] = x;
			((float*) a.cache)[at + a.kv_rank + c + half] = y;
		} else {
			((__nv_bfloat16*) a.cache)[at + a.kv_rank + c] = __float2bfloat16_rn(x);
			((__nv_bfloat16*) a.cache)[at + a.kv_rank + c + half] = __float2bfloat16_rn(y);
		}
	}
}
static inline int launch_latent_post(const LatentPostArgs& a, int rows, cudaStream_t s) {
	if (a.rot % 2 || (a.rot && !a.freq)) return set_error(XALM_ERR_INVALID, "latent_post: %d rotated columns", a.rot);
	const int widest = std::max(a.q_rank, a.kv_rank);
	latent_post_kernel<<<rows, widest >= 512 ? 256 : widest >= 128 ? 128 : 64, 0, s>>>(a);
	return launch_check("latent_post");
}

struct RopeHeadsArgs {
	const float* src; // (T, lds): head h at columns src_off + h * src_stride
	float* dst;       // (T, ldd): head h at columns dst_off + h * dst_stride; may be src (then nothing but the rotated entries is written)
	int lds, src_off, src_stride, ldd, dst_off, dst_stride;
	int heads, n;     // entries of a head that travel: the first 2 * rot_half rotated, the rest copied
	int rot_half;
	const float* freq; // (rot_half)
	const SeqStep* step;
};
// grid (tokens, ceil(heads / 8)), 256 threads: a warp per head
static __global__ void rope_heads_kernel(RopeHeadsArgs a) {
	const int t = blockIdx.x, lane = threadIdx.x & 31, h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
	if (t >= a.step->n || h >= a.heads) return;
	const float pos = (float) (a.step->pos0 + t);
	const float* s = a.src + (size_t) t * a.lds + a.src_off + (size_t) h * a.src_stride;
	float* d = a.dst + (size_t) t * a.ldd + a.dst_off + (size_t) h * a.dst_stride;
	const int r = a.rot_half;
	for (int c = lane; c < r; c += 32) {
		float sn, cs;
		sincosf(pos * a.freq[c], &sn, &cs);
		const float u = s[c], v = s[c + r];
		d[c] = u * cs - v * sn;
		d[c + r] = v * cs + u * sn;
	}
	if (d != s)
		for (int c = 2 * r + lane; c < a.n; c += 32) d[c] = s[c];
}
static inline int launch_rope_heads(const RopeHeadsArgs& a, int rows, cudaStream_t s) {
	if (a.rot_half < 0 || 2 * a.rot_half > a.n || (a.rot_half && !a.freq)) return set_error(XALM_ERR_INVALID, "rope_heads: %d pairs in a head of %d", a.rot_half, a.n);
	rope_heads_kernel<<<dim3(rows, (a.heads + 7) / 8), 256, 0, s>>>(a);
	return launch_check("rope_heads");
}

} // namespace mix
} // namespace xalm
