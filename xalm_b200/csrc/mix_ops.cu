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

extern "C" {

int xalm_cuda_swa_attention(float* out, const float* q, const float* gate, const float* k, const float* v, int T, int pos0, int H, int G, int d, int dv,
                            int window, float scale, float softcap, const float* r1, const float* r2, const float* talk, int ring, int n_splits,
                            int cache_bf16) {
	if (!out || !q || !k || !v || T <= 0 || pos0 < 0 || H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0 || window <= 0 || n_splits < 1)
		return set_error(XALM_ERR_INVALID, "swa_attention: bad argument");
	const int n = pos0 + T;
	const long long need = std::min<long long>(n, (long long) window - 1 + T);
	if (ring < need) return set_error(XALM_ERR_INVALID, "swa_attention: a ring of %d slots cannot hold %lld live positions", ring, need);
	if (!r1 != !r2) return set_error(XALM_ERR_INVALID, "swa_attention: r1 and r2 come together");
	const size_t smem = swa_smem_bytes(H, d, dv);
	if (!swa_pick_tq(H, G, d, dv, T) && smem > 200 * 1024) return set_error(XALM_ERR_UNSUPPORTED, "swa_attention: heads need %zu bytes of shared memory", smem);
	Pool pool;
	// the ring as the cache manager leaves it: position p lives in slot p % ring, older positions are overwritten
	const size_t esz = cache_bf16 ? 2 : 4;
	std::vector<uint8_t> kr((size_t) ring * G * d * esz, 0), vr((size_t) ring * G * dv * esz, 0);
	for (int p = 0; p < n; p++) {
		const int slot = p % ring;
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
	a.ring = ring; a.H = H; a.G = G; a.d = d; a.dv = dv; a.window = window; a.scale = scale; a.softcap = softcap;
	a.r1 = pool.put(r1, (size_t) H); a.r2 = pool.put(r2, (size_t) H); a.talk = pool.put(talk, (size_t) H * H);
	a.step = pool.put(&st, 1);
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

} // extern "C"
