// moe_ops.cuh — a mixture of small gated feed-forward experts, as three mechanisms that another design can use on their own:
//
//   moe_router_kernel   per token: logits z = W_router h in fp32, scores s = sigmoid(z); optionally the experts form n_groups equal groups
//                       of neighbours, a group scores the sum of its two largest s, and only experts of the keep_groups best groups can be
//                       chosen; the `top` largest s among those are chosen (ties: the lower index), their weights are the scores
//                       themselves (not renormalised)
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
};

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
		for (int k = lane; k < a.K; k += 32) z = fmaf(ldf(W + (size_t) e * a.K + k), hs[k], z);
		z = warp_sum(z);
		if (lane == 0) sc[e] = sigmoidf_(z);
	}
	__syncthreads();
	if (warp != 0) return;
	const int ng = a.n_groups > 1 ? a.n_groups : 1, gsz = a.E / ng;
	if (ng > 1) {
		for (int g = lane; g < ng; g += 32) { // sum of the group's two largest scores
			float m1 = -INFINITY, m2 = -INFINITY;
			for (int j = 0; j < gsz; j++) {
				const float v = sc[g * gsz + j];
				if (v > m1) { m2 = m1; m1 = v; }
				else if (v > m2) m2 = v;
			}
			gsc[g] = gsz > 1 ? m1 + m2 : m1;
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
}

constexpr int MOE_TM = 64; // rows of a tile

struct MoeSortArgs {
	const int* idx; // (T, top)
	int top, E;
	const SeqStep* step;
	int* sorted;  // (T * top) pair ids, expert after expert
	int* tiles;   // (max_tiles, 3): expert, first place in `sorted`, rows
	int* n_tiles; // (1)
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
		*a.n_tiles = nt;
	}
	__syncthreads();
	for (int e = tid; e < a.E; e += nth) cnt[e] = off[e]; // cursors
	__syncthreads();
	for (int p = tid; p < P; p += nth) a.sorted[atomicAdd(&cnt[a.idx[p]], 1)] = p; // the order inside an expert does not matter: rows are independent
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
static inline int launch_moe_gemm(const MoeGemmArgs& a, bool w_bf16, int pairs, int E, cudaStream_t s) {
	const dim3 grid((a.N + 63) / 64, moe_max_tiles(pairs, E));
	if (w_bf16) moe_gemm_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(a);
	else moe_gemm_kernel<float><<<grid, 256, 0, s>>>(a);
	return launch_check("moe_gemm");
}

} // namespace mix
} // namespace xalm
