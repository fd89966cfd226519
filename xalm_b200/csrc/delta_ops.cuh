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
// A column of S evolves on its own (u_c needs only S[:, c]), so a thread owns one column: its d values sit in registers (d <= 128) or in
// shared memory, k and q of the token are broadcast from shared memory, and nothing is reduced across threads until the per-head norm.
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

__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }

static __global__ void delta_prep_kernel(DeltaArgs a) {
	extern __shared__ float sm[]; // 2 G d: q and k after convolution and silu
	const int t = blockIdx.x, tid = threadIdx.x, nth = blockDim.x, lane = tid & 31, warp = tid >> 5, nw = nth >> 5;
	if (t >= a.step->n) return;
	const int nq = a.G * a.d, nv = a.H * a.dv, Cc = 2 * nq + nv, taps = a.taps;
	float* prow = a.prep + (size_t) t * a.ldp;
	for (int cc = tid; cc < Cc; cc += nth) {
		const int sec = cc < nq ? 0 : cc < 2 * nq ? 1 : 2, lc = cc - (sec == 0 ? 0 : sec == 1 ? nq : 2 * nq);
		const int off = sec == 0 ? a.q_off : sec == 1 ? a.k_off : a.v_off;
		const float* w = (sec == 0 ? a.wq : sec == 1 ? a.wk : a.wv) + (size_t) lc * taps;
		float y = 0.f;
		for (int tau = 0; tau < taps; tau++) {
			const int r = t - (taps - 1) + tau; // row of this step, or (negative) one of the positions before it
			const float x = r >= 0 ? a.proj[(size_t) r * a.ld + off + lc] : a.conv_state[(size_t) (taps - 1 + r) * Cc + cc];
			y = fmaf(w[tau], x, y);
		}
		y = y * sigmoidf_(y);
		if (sec == 2) prow[cc] = y;
		else sm[cc] = y;
	}
	__syncthreads();
	for (int hd = warp; hd < 2 * a.G; hd += nw) { // q heads, then k heads
		const float* x = sm + (size_t) hd * a.d;
		float ss = 0.f;
		for (int c = lane; c < a.d; c += 32) ss = fmaf(x[c], x[c], ss);
		ss = warp_sum(ss);
		const float r = (hd < a.G ? a.q_scale : 1.f) / sqrtf(ss + a.unit_eps);
		for (int c = lane; c < a.d; c += 32) prow[(size_t) hd * a.d + c] = x[c] * r;
	}
	for (int h = tid; h < a.H; h += nth) {
		const float* row = a.proj + (size_t) t * a.ld;
		prow[Cc + h] = sigmoidf_(row[a.b_off + h]);
		prow[Cc + a.H + h] = expf(-expf(a.A_log[h]) * softplusf_(row[a.a_off + h] + a.dt_bias[h]));
	}
}

constexpr int DELTA_TT = 16; // tokens staged at a time

// D > 0: a thread keeps its column of the state in D registers (d <= D); D == 0: in shared memory (any d that fits)
template <int D>
__global__ void delta_rule_kernel(DeltaArgs a) {
	extern __shared__ __align__(16) float sm[];
	const int h = blockIdx.x, tid = threadIdx.x, nth = blockDim.x, lane = tid & 31, warp = tid >> 5, nw = nth >> 5;
	const int d = a.d, dv = a.dv, dp = D > 0 ? D : ((d + 3) & ~3), hk = h / (a.H / a.G);
	const int nq = a.G * d, Cc = 2 * nq + a.H * dv;
	float* ks = sm;                         // TT * dp
	float* qs = ks + DELTA_TT * dp;         // TT * dp
	float* vs = qs + DELTA_TT * dp;         // TT * dv
	float* och = vs + DELTA_TT * dv;        // TT * dv
	float* bg = och + DELTA_TT * dv;        // TT * 2: beta, g
	float* Ssh = bg + DELTA_TT * 2;         // D == 0: dp * nth
	const int T = a.step->n;
	const int c = tid; // this thread's column
	const bool live = c < dv;
	float* st = a.state + (size_t) h * d * dv;
	float S[D > 0 ? D : 1];
	if constexpr (D > 0) {
#pragma unroll
		for (int i = 0; i < (D > 0 ? D : 1); i++) S[i] = (live && i < d) ? st[(size_t) i * dv + c] : 0.f;
	} else {
		for (int i = 0; i < dp; i++) Ssh[(size_t) i * nth + tid] = (live && i < d) ? st[(size_t) i * dv + c] : 0.f;
	}
	for (int t0 = 0; t0 < T; t0 += DELTA_TT) {
		const int nt = min(DELTA_TT, T - t0);
		__syncthreads(); // the last tile's readers are done
		for (int x = tid; x < nt * dp; x += nth) {
			const int tt = x / dp, i = x % dp;
			const float* prow = a.prep + (size_t) (t0 + tt) * a.ldp;
			ks[x] = i < d ? prow[nq + hk * d + i] : 0.f;
			qs[x] = i < d ? prow[hk * d + i] : 0.f;
		}
		for (int x = tid; x < nt * dv; x += nth) {
			const int tt = x / dv, cc = x % dv;
			vs[x] = a.prep[(size_t) (t0 + tt) * a.ldp + 2 * nq + h * dv + cc];
		}
		for (int x = tid; x < nt * 2; x += nth) {
			const int tt = x >> 1, w = x & 1;
			bg[x] = a.prep[(size_t) (t0 + tt) * a.ldp + Cc + w * a.H + h];
		}
		__syncthreads();
		if (live) {
			for (int tt = 0; tt < nt; tt++) {
				const float beta = bg[2 * tt], g = bg[2 * tt + 1], v = vs[tt * dv + c];
				const float4* k4 = reinterpret_cast<const float4*>(ks + tt * dp);
				const float4* q4 = reinterpret_cast<const float4*>(qs + tt * dp);
				float o;
				if constexpr (D > 0) {
					float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
					for (int i = 0; i < (D > 0 ? D : 4); i += 4) {
						const float4 kk = k4[i >> 2];
						S[i] *= g; S[i + 1] *= g; S[i + 2] *= g; S[i + 3] *= g;
						d0 = fmaf(kk.x, S[i], d0); d1 = fmaf(kk.y, S[i + 1], d1); d2 = fmaf(kk.z, S[i + 2], d2); d3 = fmaf(kk.w, S[i + 3], d3);
					}
					const float u = beta * (v - ((d0 + d1) + (d2 + d3)));
					float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
					for (int i = 0; i < (D > 0 ? D : 4); i += 4) {
						const float4 kk = k4[i >> 2], qq = q4[i >> 2];
						S[i] = fmaf(kk.x, u, S[i]); S[i + 1] = fmaf(kk.y, u, S[i + 1]); S[i + 2] = fmaf(kk.z, u, S[i + 2]); S[i + 3] = fmaf(kk.w, u, S[i + 3]);
						o0 = fmaf(qq.x, S[i], o0); o1 = fmaf(qq.y, S[i + 1], o1); o2 = fmaf(qq.z, S[i + 2], o2); o3 = fmaf(qq.w, S[i + 3], o3);
					}
					o = (o0 + o1) + (o2 + o3);
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
				och[tt * dv + c] = o;
			}
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
			const float* grow = a.proj + (size_t) (t0 + tt) * a.ld + a.g_off + h * dv;
			float* orow = a.out + (size_t) (t0 + tt) * (a.H * dv) + h * dv;
			for (int cc = lane; cc < dv; cc += 32) {
				const float z = grow[cc];
				orow[cc] = och[tt * dv + cc] * r * (a.norm_w ? a.norm_w[cc] : 1.f) * (z * sigmoidf_(z));
			}
		}
	}
	if (live) {
		if constexpr (D > 0) {
#pragma unroll
			for (int i = 0; i < (D > 0 ? D : 1); i++)
				if (i < d) st[(size_t) i * dv + c] = S[i];
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

static inline int delta_threads(int dv) { return (dv + 31) / 32 * 32; }
// the register tile for a head of d x dv: 0 (shared memory) when d is beyond 128 or the CTA's dv threads would not fit the register file
static inline int delta_reg_dim(int d, int dv) {
	const int D = d <= 32 ? 32 : d <= 64 ? 64 : d <= 128 ? 128 : 0;
	return D && (size_t) delta_threads(dv) * (D + 56) <= 65536 ? D : 0;
}
static inline size_t delta_rule_smem(int d, int dv) {
	const int D = delta_reg_dim(d, dv), dp = D ? D : ((d + 3) & ~3);
	return sizeof(float) * ((size_t) DELTA_TT * (2 * dp + 2 * dv + 2) + (D ? 0 : (size_t) dp * delta_threads(dv)));
}
static inline bool delta_ok(int d, int dv) { return dv <= 1024 && delta_rule_smem(d, dv) <= 200 * 1024; }
static inline int delta_prepare(int d, int dv) { // outside a stream capture
	if (delta_rule_smem(d, dv) > 48 * 1024) {
		const int D = delta_reg_dim(d, dv);
		const void* f = D == 32 ? (const void*) delta_rule_kernel<32> : D == 64 ? (const void*) delta_rule_kernel<64> : D == 128 ? (const void*) delta_rule_kernel<128>
		                                                                                                                       : (const void*) delta_rule_kernel<0>;
		XALM_CUDA_CHECK(cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
	}
	return XALM_OK;
}
// rows: tokens of the step (host-side bound); two launches
static inline int launch_delta(const DeltaArgs& a, int rows, cudaStream_t s) {
	if (a.H % a.G || a.taps < 1 || !delta_ok(a.d, a.dv)) return set_error(XALM_ERR_UNSUPPORTED, "delta rule: heads %d / %d, state %d x %d", a.H, a.G, a.d, a.dv);
	const size_t psm = (size_t) 2 * a.G * a.d * 4;
	if (psm > 48 * 1024) return set_error(XALM_ERR_UNSUPPORTED, "delta rule: %d key channels do not fit shared memory", a.G * a.d);
	delta_prep_kernel<<<rows, 256, psm, s>>>(a);
	XALM_TRY(launch_check("delta_prep"));
	const int nth = delta_threads(a.dv), D = delta_reg_dim(a.d, a.dv);
	const size_t smem = delta_rule_smem(a.d, a.dv);
	if (D == 32) delta_rule_kernel<32><<<a.H, nth, smem, s>>>(a);
	else if (D == 64) delta_rule_kernel<64><<<a.H, nth, smem, s>>>(a);
	else if (D == 128) delta_rule_kernel<128><<<a.H, nth, smem, s>>>(a);
	else delta_rule_kernel<0><<<a.H, nth, smem, s>>>(a);
	return launch_check("delta_rule");
}

} // namespace mix
} // namespace xalm
