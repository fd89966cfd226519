// nabalix.cu — the Nabalix family of the model registry (family.h): a decoder-only model described by a config.json whose
// layers run two token mixers side by side on the same normed input — windowed softmax attention (grouped K/V heads, soft-capped
// scores, logarithmic distance bias, score mixing across heads, sigmoid output gate) and an HGRN2 gated linear recurrence — join
// them as the mean of their RMS-normed outputs, follow with a clamped-GLU feed-forward, and carry the residual in several
// hyper-connected streams with a layer scale on every sublayer.
//
// One step function serves prompts and generation (seq_step): n tokens of the running sequence, cut into passes of at most
// "seq_chunk" positions.  Per pass and layer:
//     hc_norm                      u = sum_s in[s] x_s -> RMS norm (1 + w)
//     rows product [in-projection] one matrix [Lq | Lg | Rq | Rf | Rv | Lk | Lv]; the K/V columns go straight into the ring cache
//     swa_attn (+ swa_merge)       left mixer, gate fused;   hgrn2: right mixer, activations + per-head norm fused
//     rows product x 2             the two output projections
//     dual_norm_hc                 1/2 (norm + norm), layer scale, hyper-connection write
//     hc_norm, rows product [gate|up interleaved, GLU fused], rows product [down, layer scale + hyper-connection write fused]
// One-token steps replay a captured CUDA graph (position and token are read from device memory).
//
// Cache / state manager: per layer a K/V ring of min(max_tokens, window - 1 + seq_chunk) slots (slot = position mod ring: a pass
// needs its own keys and the window - 1 before them at once) and the fp32 recurrent state (heads x dim x vdim).  release() hands
// both back: the state is zeroed, the position returns to 0.
//
// Precision: XALM_PRECISION_F32 computes everything in IEEE fp32 (weights are widened, the K/V ring holds fp32).  XALM_PRECISION_BF16
// keeps weights and K/V ring in bf16 and routes batched matrix products whose shapes allow it through the tcgen05 GEMM of
// prefill.cu (fp16 hi+lo operand pairs, fp32 accumulation); norms, scores, softmax, gates, the recurrence and the streams stay fp32.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <string>
#include <vector>

#define XALM_SECONDARY_TU
#include "common.cuh"
#include "family.h"
#include "formats.cuh"
#include "host/json.h"
#include "mix_ops.cuh"
#include "prefill.h"

namespace xalm {
namespace {

using namespace mix;

struct LeftCfg {
	int H = 0, G = 0, d = 0, dv = 0, window = 0; // window 0: every earlier position is visible
	float scale = 1.f, softcap = 0.f;
};
struct RightCfg {
	int H = 0, d = 0, dv = 0;
};

// a tensor as uploaded: fp32 on the host until finalize builds the device layouts
struct HostTensor {
	std::vector<int> shape;
	bool required = true;
	bool matrix = false;
	bool got = false;
	int type = 0;
	std::vector<float> v;
};

struct Layer {
	LeftCfg L;
	RightCfg R;
	bool has_mlp = false;
	int ff = 0;
	float limit = 0.f;
	// device
	void* w_in = nullptr;   // [Lq | Lg | Rq | Rf | Rv | Lk | Lv] x width
	void* w_lo = nullptr;   // width x (H dv)
	void* w_ro = nullptr;   // width x (Hr dvr)
	void* w_gu = nullptr;   // (2 ff) x width, gate and up rows interleaved
	void* w_down = nullptr; // width x ff
	WMat m_in, m_lo, m_ro, m_gu, m_down; // the same buffers as the tensor-core path's operand descriptors
	TcWeight t_in, t_lo, t_ro, t_gu, t_down; // resident fp16 operand tiles for passes of many tokens (16-bit mode)
	int n_in = 0, n_plain = 0, off_lq = 0, off_lg = 0, off_rq = 0, off_rf = 0, off_rv = 0;
	bool has_gate = false;
	float *norm1 = nullptr, *norm2 = nullptr, *r1 = nullptr, *r2 = nullptr, *talk = nullptr, *fb = nullptr, *lower = nullptr, *rnorm = nullptr;
	float *lout = nullptr, *rout = nullptr, *ls1 = nullptr, *ls2 = nullptr;
	float *hc_in[2] = {nullptr, nullptr}, *hc_out[2] = {nullptr, nullptr}, *hc_mix[2] = {nullptr, nullptr};
	void *kc = nullptr, *vc = nullptr;
	int ring = 0;
	float* state = nullptr;
};

} // namespace
} // namespace xalm

using namespace xalm;
using namespace xalm::mix;

struct NabalixModel { // what a Nabalix handle points to (ModelHead first)
	ModelHead head = {nullptr};
	int device = 0, precision = XALM_PRECISION_BF16, max_tokens = 0;
	int vocab = 0, width = 0, S = 1;
	float eps = 1e-5f;
	std::vector<Layer> layers;
	std::map<std::string, HostTensor> tensors;
	std::vector<std::string> order; // expected tensors in file order
	bool w_bf16 = true;             // matrices live on the device as bf16 (else fp32)
	bool finalized = false;
	std::vector<void*> allocs;
	void *embed = nullptr, *w_head = nullptr;
	WMat m_head;
	TcWeight t_head;
	uint8_t *a_hi = nullptr, *a_lo = nullptr; // activation operand planes of the tensor-core path
	float* tc_out = nullptr;                  // its plain fp32 product, when an epilogue follows
	int tc_min_rows = 32;
	float* final_norm = nullptr;
	// activations of one pass
	int chunk = 256;
	float *xs = nullptr, *h = nullptr, *proj = nullptr, *att = nullptr, *ro = nullptr, *ol = nullptr, *orr = nullptr, *y = nullptr, *logits = nullptr;
	float *part_o = nullptr, *part_ml = nullptr, *layer_sums = nullptr;
	unsigned* tickets = nullptr; // per query tile: arrivals of the attention's key splits
	int graph_launches[2] = {0, 0};    // kernels in the captured one-token step (without / with logits)
	int part_cap = 0, keep_layers = 0; // part_cap: (token, key split) pairs the attention's partial buffers hold
	int* d_tokens = nullptr;
	SeqStep* d_step = nullptr;
	float* h_logits = nullptr; // pinned, chunk x vocab
	size_t proj_ld = 0;
	cudaStream_t stream = nullptr, own_stream = nullptr;
	cudaStream_t side = nullptr;                  // the recurrence of a layer runs here, beside the attention on `stream`
	cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
	cudaGraphExec_t graph[2] = {nullptr, nullptr};
	int pos = 0; // tokens the running sequence holds
	int last_launches = 0;
	bool use_tc = false;
	long long weight_bytes = 0, weight_bytes_tc = 0;
};

namespace xalm {
namespace {

typedef NabalixModel Nb;

// ---- config.json ------------------------------------------------------------------------------------------------------------
int geti(const xjson::Value& o, const char* k) {
	const xjson::Value& v = o.at(k);
	if (v.kind != xjson::Value::Number) throw std::invalid_argument(std::string("config: '") + k + "' is not a number");
	return (int) v.num;
}
void expect(Nb* m, const std::string& name, std::vector<int> shape, bool matrix, bool required = true) {
	HostTensor t;
	t.shape = std::move(shape);
	t.matrix = matrix;
	t.required = required;
	m->tensors.emplace(name, std::move(t));
	m->order.push_back(name);
}

int parse_config(Nb* m, const char* json) {
	try {
		const xjson::Value c = xjson::Parser::parse(json, strlen(json));
		m->vocab = geti(c, "vocab");
		m->width = geti(c, "width");
		m->S = c.contains("streams") ? geti(c, "streams") : 1;
		if (const xjson::Value* nv = c.find("norm"))
			if (const xjson::Value* e = nv->find("eps")) m->eps = (float) e->num;
		if (m->vocab <= 0 || m->width <= 0) return set_error(XALM_ERR_INVALID, "config: vocab / width must be positive");
		if (m->S < 1 || m->S > MAX_STREAMS) return set_error(XALM_ERR_UNSUPPORTED, "config: %d streams (1..%d)", m->S, MAX_STREAMS);
		const int W = m->width, S = m->S;
		expect(m, "embed", {m->vocab, W}, true);
		const xjson::Value& layers = c.at("layers");
		if (layers.kind != xjson::Value::Array || layers.arr.empty()) return set_error(XALM_ERR_INVALID, "config: no layers");
		for (size_t li = 0; li < layers.arr.size(); li++) {
			const xjson::Value& lv = layers.arr[li];
			const std::string type = lv.at("type").str;
			if (type != "parallel") return set_error(XALM_ERR_UNSUPPORTED, "config: layer %zu has mixer type '%s' (this family runs 'parallel')", li, type.c_str());
			Layer L;
			const xjson::Value& mx = lv.at("mixer");
			const xjson::Value& lf = mx.at("left");
			L.L.H = geti(lf, "heads");
			L.L.G = lf.contains("kv_heads") ? geti(lf, "kv_heads") : L.L.H;
			L.L.d = geti(lf, "dim");
			L.L.dv = lf.contains("vdim") ? geti(lf, "vdim") : L.L.d;
			L.L.scale = lf.contains("scale") ? (float) lf.at("scale").num : 1.f / sqrtf((float) L.L.d);
			L.L.softcap = lf.contains("softcap") ? (float) lf.at("softcap").num : 0.f;
			if (const xjson::Value* mk = lf.find("mask"))
				if (mk->kind == xjson::Value::Obj && mk->contains("size")) L.L.window = geti(*mk, "size");
			const xjson::Value& rt = mx.at("right");
			L.R.H = geti(rt, "heads");
			L.R.d = geti(rt, "dim");
			L.R.dv = rt.contains("vdim") ? geti(rt, "vdim") : L.R.d;
			if (L.L.H <= 0 || L.L.G <= 0 || L.L.H % L.L.G || L.L.d <= 0 || L.L.dv <= 0 || L.L.window < 0)
				return set_error(XALM_ERR_INVALID, "config: layer %zu: bad attention sizes", li);
			if (L.R.H <= 0 || L.R.d <= 0 || L.R.dv <= 0) return set_error(XALM_ERR_INVALID, "config: layer %zu: bad recurrence sizes", li);
			if (L.R.dv > 1024) return set_error(XALM_ERR_UNSUPPORTED, "config: layer %zu: recurrence vdim %d (at most 1024)", li, L.R.dv);
			const xjson::Value* mlp = lv.find("mlp");
			if (mlp && mlp->kind == xjson::Value::Obj) {
				const std::string kind = mlp->contains("kind") ? mlp->at("kind").str : "dense";
				if (kind != "dense") return set_error(XALM_ERR_UNSUPPORTED, "config: layer %zu has feed-forward kind '%s'", li, kind.c_str());
				L.has_mlp = true;
				L.ff = geti(*mlp, "ff");
				L.limit = mlp->contains("limit") ? (float) mlp->at("limit").num : INFINITY;
				if (L.ff <= 0) return set_error(XALM_ERR_INVALID, "config: layer %zu: ff", li);
			}
			const std::string p = "l" + std::to_string(li) + ".";
			const int H = L.L.H, G = L.L.G, d = L.L.d, dv = L.L.dv, Hr = L.R.H, dr = L.R.d, dvr = L.R.dv;
			expect(m, p + "norm1", {W}, false);
			if (L.has_mlp) expect(m, p + "norm2", {W}, false);
			expect(m, p + "mix.left.q", {H * d, W}, true);
			expect(m, p + "mix.left.k", {G * d, W}, true);
			expect(m, p + "mix.left.v", {G * dv, W}, true);
			expect(m, p + "mix.left.r1", {H}, false, false);
			expect(m, p + "mix.left.r2", {H}, false, false);
			expect(m, p + "mix.left.talk", {H, H}, false, false);
			expect(m, p + "mix.left.g", {H * dv, W}, true, false);
			expect(m, p + "mix.left.o", {W, H * dv}, true);
			expect(m, p + "mix.right.q", {Hr * dr, W}, true);
			expect(m, p + "mix.right.f", {Hr * dr, W}, true);
			expect(m, p + "mix.right.f.b", {Hr * dr}, false, false);
			expect(m, p + "mix.right.lower", {Hr * dr}, false, false);
			expect(m, p + "mix.right.v", {Hr * dvr, W}, true);
			expect(m, p + "mix.right.norm", {dvr}, false, false);
			expect(m, p + "mix.right.o", {W, Hr * dvr}, true);
			expect(m, p + "mix.left.out", {W}, false);
			expect(m, p + "mix.right.out", {W}, false);
			if (L.has_mlp) {
				expect(m, p + "mlp.gate", {L.ff, W}, true);
				expect(m, p + "mlp.up", {L.ff, W}, true);
				expect(m, p + "mlp.down", {W, L.ff}, true);
			}
			expect(m, p + "ls1", {W}, false, false);
			if (L.has_mlp) expect(m, p + "ls2", {W}, false, false);
			for (int q = 1; q <= (L.has_mlp ? 2 : 1); q++) {
				const std::string hp = p + "hc" + std::to_string(q) + ".";
				expect(m, hp + "in", {S}, false, S > 1);
				expect(m, hp + "out", {S}, false, S > 1);
				expect(m, hp + "mix", {S, S}, false, S > 1);
			}
			m->layers.push_back(L);
		}
		expect(m, "final.norm", {W}, false);
		expect(m, "head", {m->vocab, W}, true);
	} catch (const std::exception& e) {
		return set_error(XALM_ERR_INVALID, "config.json: %s", e.what());
	}
	return XALM_OK;
}

// ---- device memory ------------------------------------------------------------------------------------------------------------
template <typename T>
int dev_alloc(Nb* m, T** p, size_t count, bool zero = false) {
	void* q = nullptr;
	const size_t bytes = std::max<size_t>(count * sizeof(T), 16);
	cudaError_t e = cudaMalloc(&q, bytes);
	if (e != cudaSuccess) return set_error(XALM_ERR_CUDA, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
	m->allocs.push_back(q);
	if (zero) XALM_CUDA_CHECK(cudaMemset(q, 0, bytes));
	*p = reinterpret_cast<T*>(q);
	return XALM_OK;
}

int upload_vec(Nb* m, const std::string& name, float** dst) {
	*dst = nullptr;
	const HostTensor& t = m->tensors.at(name);
	if (!t.got) return XALM_OK;
	XALM_TRY(dev_alloc(m, dst, t.v.size()));
	XALM_CUDA_CHECK(cudaMemcpy(*dst, t.v.data(), t.v.size() * 4, cudaMemcpyHostToDevice));
	m->weight_bytes += (long long) t.v.size() * 4;
	return XALM_OK;
}

uint16_t f32_to_bf16_bits(float f) {
	uint32_t u;
	memcpy(&u, &f, 4);
	if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t) ((u >> 16) | 0x40);
	u += 0x7fffu + ((u >> 16) & 1u);
	return (uint16_t) (u >> 16);
}

// rows of several host matrices, one after the other (interleave: rows of the two parts alternate), as one device matrix
int upload_rows(Nb* m, const std::vector<const HostTensor*>& parts, int K, bool interleave, void** dst, WMat* wm) {
	size_t rows = 0;
	for (const HostTensor* t : parts) rows += t ? (size_t) t->shape[0] : 0;
	const size_t esz = m->w_bf16 ? 2 : 4;
	std::vector<uint8_t> buf(rows * (size_t) K * esz);
	size_t r = 0;
	auto put_row = [&](const float* src) {
		if (m->w_bf16) {
			uint16_t* o = reinterpret_cast<uint16_t*>(buf.data()) + r * (size_t) K;
			for (int k = 0; k < K; k++) o[k] = f32_to_bf16_bits(src[k]);
		} else memcpy(buf.data() + r * (size_t) K * 4, src, (size_t) K * 4);
		r++;
	};
	if (interleave) {
		for (int i = 0; i < parts[0]->shape[0]; i++)
			for (const HostTensor* t : parts) put_row(t->v.data() + (size_t) i * K);
	} else {
		for (const HostTensor* t : parts)
			if (t)
				for (int i = 0; i < t->shape[0]; i++) put_row(t->v.data() + (size_t) i * K);
	}
	uint8_t* d = nullptr;
	XALM_TRY(dev_alloc(m, &d, buf.size() + 64));
	XALM_CUDA_CHECK(cudaMemcpy(d, buf.data(), buf.size(), cudaMemcpyHostToDevice));
	*dst = d;
	m->weight_bytes += (long long) buf.size();
	if (wm) {
		*wm = WMat();
		wm->type = m->w_bf16 ? XALM_BF16 : XALM_F32;
		wm->rows = (int) rows;
		wm->n = K;
		wm->p0 = d;
		wm->s0 = (size_t) K * esz;
	}
	return XALM_OK;
}

// ---- row products -------------------------------------------------------------------------------------------------------------
// Passes of few tokens and the fp32 mode: the fp32 FMA kernels of mix_ops.cuh with the epilogue fused.  Passes of tc_min_rows tokens
// or more in the 16-bit mode: the tcgen05 GEMM of prefill.cu on the weight's resident fp16 tiles (activations packed to fp16, one
// plane, or hi + lo with "seq_tc" = 2), fp32 accumulation, then the same epilogue as an elementwise kernel.
int rows_product(Nb* m, const float* A, int lda, const void* W, const TcWeight* tw, int T, int N, int K, const RowsEpi& e, int* nl) {
	if (m->use_tc && tw && tw->hi && T >= m->tc_min_rows && lda == K) {
		if (e.kind == EPI_STORE && e.ldo % 4 == 0) {
			*nl += 2;
			return tc_gemm(*tw, A, T, e.out, e.ldo, m->a_hi, m->a_lo, m->stream);
		}
		*nl += 3;
		XALM_TRY(tc_gemm(*tw, A, T, m->tc_out, N, m->a_hi, m->a_lo, m->stream));
		return launch_rows_epilogue(m->tc_out, N, T, N, e, m->stream);
	}
	(*nl)++;
	return launch_rows(A, lda, W, m->w_bf16, T, N, K, e, m->stream);
}

#define NB_LAUNCH_CHECK(what)                                                                                       \
	do {                                                                                                            \
		(*nl)++;                                                                                                    \
		cudaError_t e_ = cudaGetLastError();                                                                        \
		if (e_ != cudaSuccess) return set_error(XALM_ERR_CUDA, what " launch failed: %s", cudaGetErrorString(e_));   \
	} while (0)

// hyper-connection write of sublayer q of layer L as an epilogue
RowsEpi hc_epi(Nb* m, const Layer& L, int q) {
	RowsEpi e;
	e.kind = EPI_HC;
	e.xs = m->xs;
	e.S = m->S;
	e.stream_stride = (size_t) m->chunk * m->width;
	e.hmix = L.hc_mix[q];
	e.hout = L.hc_out[q];
	e.scale = q == 0 ? L.ls1 : L.ls2;
	return e;
}

// the kernels of one pass: n tokens (ids in d_tokens, position in d_step).  want: 0 no logits, 1 the last row's, 2 every row's.
int enqueue_pass(Nb* m, int n, int want, int* nl) {
	cudaStream_t s = m->stream;
	const int W = m->width, S = m->S;
	const size_t sstride = (size_t) m->chunk * W;
	const int rt = norm_threads(W);
	if (m->w_bf16) embed_streams_kernel<__nv_bfloat16><<<n, rt, 0, s>>>((const __nv_bfloat16*) m->embed, m->d_tokens, W, S, sstride, m->xs);
	else embed_streams_kernel<float><<<n, rt, 0, s>>>((const float*) m->embed, m->d_tokens, W, S, sstride, m->xs);
	NB_LAUNCH_CHECK("embed");
	for (size_t li = 0; li < m->layers.size(); li++) {
		const Layer& L = m->layers[li];
		const int H = L.L.H, G = L.L.G, d = L.L.d, dv = L.L.dv, Hr = L.R.H, dr = L.R.d, dvr = L.R.dv;
		// ---- mixer ----
		XALM_TRY(launch_hc_norm(m->xs, S, sstride, L.hc_in[0], L.norm1, 1, m->eps, W, m->h, nullptr, n, s));
		(*nl)++;
		RowsEpi ein;
		ein.kind = EPI_SPLIT_KV;
		ein.out = m->proj;
		ein.ldo = (int) m->proj_ld;
		ein.n_plain = L.n_plain; ein.kdim = G * d; ein.vdim = G * dv; ein.ring = L.ring;
		ein.cache_f32 = m->precision == XALM_PRECISION_F32;
		ein.kc = L.kc; ein.vc = L.vc; ein.step = m->d_step;
		ein.silu_off = L.off_rq; ein.silu_n = Hr * dr; ein.gate_off = L.off_rf; ein.gate_n = Hr * dr; ein.gate_bias = L.fb; ein.gate_lower = L.lower;
		XALM_TRY(rows_product(m, m->h, W, L.w_in, &L.t_in, n, L.n_in, W, ein, nl));
		SwaArgs sa = {};
		sa.q = m->proj; sa.gate = L.has_gate ? m->proj : nullptr;
		sa.ldq = (int) m->proj_ld; sa.q_off = L.off_lq; sa.ldg = (int) m->proj_ld; sa.g_off = L.off_lg;
		sa.kc = L.kc; sa.vc = L.vc; sa.ring = L.ring;
		sa.H = H; sa.G = G; sa.d = d; sa.dv = dv;
		sa.window = L.L.window > 0 ? L.L.window : 0x7fffffff;
		sa.scale = L.L.scale; sa.softcap = L.L.softcap;
		sa.r1 = L.r1; sa.r2 = L.r2; sa.talk = L.talk;
		sa.step = m->d_step; sa.out = m->att;
		sa.n_splits = 0; // the launcher spreads the keys over CTAs when the step has few tokens
		sa.part_o = m->part_o; sa.part_ml = m->part_ml; sa.part_cap = m->part_cap; sa.tickets = m->tickets;
		Hgrn2Args ha = {};
		ha.proj = m->proj; ha.ld = (int) m->proj_ld; ha.q_off = L.off_rq; ha.f_off = L.off_rf; ha.v_off = L.off_rv;
		ha.H = Hr; ha.d = dr; ha.dv = dvr;
		ha.f_bias = L.fb; ha.lower = L.lower; ha.norm_w = L.rnorm; ha.eps = m->eps;
		ha.state = L.state; ha.step = m->d_step; ha.out = m->ro; ha.max_rows = m->chunk; ha.activated = 1;
		// the two mixers read the same projections and write different buffers: the recurrence runs on the side stream (a branch
		// of the graph, when the step is captured) while the attention and its output projection run here
		const bool overlap = tune("seq_overlap") != 0;
		if (overlap) {
			XALM_CUDA_CHECK(cudaEventRecord(m->ev_fork, s));
			XALM_CUDA_CHECK(cudaStreamWaitEvent(m->side, m->ev_fork, 0));
		}
		XALM_TRY(launch_hgrn2(ha, overlap ? m->side : s));
		(*nl)++;
		if (overlap) XALM_CUDA_CHECK(cudaEventRecord(m->ev_join, m->side));
		int swa_launches = 1;
		XALM_TRY(launch_swa(sa, n, m->precision == XALM_PRECISION_F32, s, &swa_launches));
		*nl += swa_launches;
		RowsEpi est;
		est.kind = EPI_STORE; est.out = m->ol; est.ldo = W;
		XALM_TRY(rows_product(m, m->att, H * dv, L.w_lo, &L.t_lo, n, W, H * dv, est, nl));
		if (overlap) XALM_CUDA_CHECK(cudaStreamWaitEvent(s, m->ev_join, 0));
		est.out = m->orr;
		XALM_TRY(rows_product(m, m->ro, Hr * dvr, L.w_ro, &L.t_ro, n, W, Hr * dvr, est, nl));
		NextRead nx; // the feed-forward's read of the streams rides along with the mixer's write when the row fits
		const bool carry = L.has_mlp && dual_norm_can_carry(W);
		if (carry) { nx.a = L.hc_in[1]; nx.w = L.norm2; nx.one_plus = 1; nx.h = m->h; }
		XALM_TRY(launch_dual_norm_hc(m->ol, m->orr, L.lout, L.rout, m->eps, W, hc_epi(m, L, 0), n, s, nx));
		(*nl)++;
		// ---- feed-forward ----
		if (L.has_mlp) {
			if (!carry) {
				XALM_TRY(launch_hc_norm(m->xs, S, sstride, L.hc_in[1], L.norm2, 1, m->eps, W, m->h, nullptr, n, s));
				(*nl)++;
			}
			RowsEpi eg;
			eg.kind = EPI_GLU; eg.out = m->y; eg.ldo = L.ff; eg.limit = L.limit;
			XALM_TRY(rows_product(m, m->h, W, L.w_gu, &L.t_gu, n, 2 * L.ff, W, eg, nl));
			XALM_TRY(rows_product(m, m->y, L.ff, L.w_down, &L.t_down, n, W, L.ff, hc_epi(m, L, 1), nl));
		}
		if (m->keep_layers) {
			XALM_TRY(launch_hc_norm(m->xs, S, sstride, nullptr, m->final_norm, 1, m->eps, W, nullptr, m->layer_sums + li * (size_t) m->chunk * W, n, s));
			(*nl)++;
		}
	}
	if (want) {
		const int rows = want == 2 ? n : 1, first = want == 2 ? 0 : n - 1;
		XALM_TRY(launch_hc_norm(m->xs + (size_t) first * W, S, sstride, nullptr, m->final_norm, 1, m->eps, W, m->h, nullptr, rows, s));
		(*nl)++;
		RowsEpi eh;
		eh.kind = EPI_STORE; eh.out = m->logits; eh.ldo = m->vocab;
		XALM_TRY(rows_product(m, m->h, W, m->w_head, &m->t_head, rows, m->vocab, W, eh, nl));
	}
	return XALM_OK;
}

int check_ready(Nb* m) {
	if (!m) return set_error(XALM_ERR_INVALID, "model is NULL");
	if (!m->finalized) return set_error(XALM_ERR_STATE, "the model is not finalized");
	XALM_CUDA_CHECK(cudaSetDevice(m->device));
	return XALM_OK;
}

int ensure_graph(Nb* m, int mode) {
	if (m->graph[mode]) return XALM_OK;
	cudaGraph_t g = nullptr;
	XALM_CUDA_CHECK(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
	int nl = 0;
	const int rc = enqueue_pass(m, 1, mode ? 1 : 0, &nl);
	cudaError_t e = cudaStreamEndCapture(m->stream, &g);
	if (rc != XALM_OK) {
		if (g) cudaGraphDestroy(g);
		return rc;
	}
	if (e != cudaSuccess) return set_error(XALM_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
	m->graph_launches[mode] = nl;
	e = cudaGraphInstantiate(&m->graph[mode], g, 0);
	cudaGraphDestroy(g);
	if (e != cudaSuccess) return set_error(XALM_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
	return XALM_OK;
}

// one pass of n <= chunk tokens at the sequence's position; the logits (want) stay on the device
int run_pass(Nb* m, const int* tokens, int n, int want) {
	for (int i = 0; i < n; i++)
		if (tokens[i] < 0 || tokens[i] >= m->vocab) return set_error(XALM_ERR_INVALID, "token %d out of range", tokens[i]);
	const SeqStep st = {m->pos, n};
	XALM_CUDA_CHECK(cudaMemcpyAsync(m->d_tokens, tokens, (size_t) n * 4, cudaMemcpyHostToDevice, m->stream));
	XALM_CUDA_CHECK(cudaMemcpyAsync(m->d_step, &st, sizeof st, cudaMemcpyHostToDevice, m->stream));
	int nl = 0;
	if (n == 1 && tune("seq_graph")) {
		const int mode = want ? 1 : 0;
		XALM_TRY(ensure_graph(m, mode));
		XALM_CUDA_CHECK(cudaGraphLaunch(m->graph[mode], m->stream));
		nl = m->graph_launches[mode]; // as counted at capture
	} else {
		XALM_TRY(enqueue_pass(m, n, want, &nl));
	}
	m->last_launches = nl;
	m->pos += n;
	return XALM_OK;
}

// the step function: n tokens of the running sequence from position pos0 (= what the sequence holds)
int seq_step(Nb* m, const int* tokens, int n, int pos0, int want, float* logits_host, const int* targets, float* probs_host) {
	XALM_TRY(check_ready(m));
	if (!tokens || n <= 0) return set_error(XALM_ERR_INVALID, "step: no tokens");
	if (want < 0 || want > 2) return set_error(XALM_ERR_INVALID, "step: want_logits = %d", want);
	if (targets && want != 2) return set_error(XALM_ERR_INVALID, "step: target probabilities need the logits of every position");
	if (pos0 != m->pos)
		return set_error(XALM_ERR_STATE, "step: position %d, but the sequence holds %d tokens (release it to start another)", pos0, m->pos);
	if ((long long) pos0 + n > m->max_tokens) return set_error(XALM_ERR_INVALID, "step: positions [%d, %d) exceed max_tokens %d", pos0, pos0 + n, m->max_tokens);
	const int V = m->vocab;
	for (int at = 0; at < n; at += m->chunk) {
		const int nc = std::min(m->chunk, n - at);
		const bool last = at + nc == n;
		const int w = want == 2 ? 2 : (want == 1 && last ? 1 : 0);
		XALM_TRY(run_pass(m, tokens + at, nc, w));
		if (w) {
			const int rows = w == 2 ? nc : 1;
			XALM_CUDA_CHECK(cudaMemcpyAsync(m->h_logits, m->logits, (size_t) rows * V * 4, cudaMemcpyDeviceToHost, m->stream));
			XALM_CUDA_CHECK(cudaStreamSynchronize(m->stream));
			if (logits_host) memcpy(logits_host + (w == 2 ? (size_t) at * V : 0), m->h_logits, (size_t) rows * V * 4);
			if (targets && probs_host)
				for (int i = 0; i < rows; i++) { // Sampler::sample_prob (sampler.cpp:18-33)
					const float* lg = m->h_logits + (size_t) i * V;
					if (targets[at + i] < 0 || targets[at + i] >= V) return set_error(XALM_ERR_INVALID, "step: target %d out of range", targets[at + i]);
					float top = lg[0];
					for (int k = 1; k < V; k++) top = std::max(top, lg[k]);
					float den = 0.f;
					for (int k = 0; k < V; k++) den += expf(lg[k] - top);
					probs_host[at + i] = expf(lg[targets[at + i]] - top) / den;
				}
		}
	}
	XALM_CUDA_CHECK(cudaStreamSynchronize(m->stream));
	return XALM_OK;
}

// ---- family table ---------------------------------------------------------------------------------------------------------------
void nb_destroy(Nb* m) {
	if (!m) return;
	cudaSetDevice(m->device);
	if (m->stream) cudaStreamSynchronize(m->stream);
	for (int i = 0; i < 2; i++)
		if (m->graph[i]) cudaGraphExecDestroy(m->graph[i]);
	for (void* p : m->allocs) cudaFree(p);
	for (Layer& L : m->layers)
		for (TcWeight* t : {&L.t_in, &L.t_lo, &L.t_ro, &L.t_gu, &L.t_down}) tc_weight_free(t);
	tc_weight_free(&m->t_head);
	if (m->h_logits) cudaFreeHost(m->h_logits);
	if (m->own_stream) cudaStreamDestroy(m->own_stream);
	if (m->side) cudaStreamDestroy(m->side);
	if (m->ev_fork) cudaEventDestroy(m->ev_fork);
	if (m->ev_join) cudaEventDestroy(m->ev_join);
	delete m;
}

extern const ModelFamily nabalix_family;

int nb_create(const char* json, int device, int max_tokens, int precision, Nb** out) {
	if (max_tokens <= 0) return set_error(XALM_ERR_INVALID, "max_tokens must be positive");
	Nb* m = new Nb();
	m->head.family = &nabalix_family;
	m->device = device;
	m->precision = precision;
	m->max_tokens = max_tokens;
	const int rc = parse_config(m, json); // before the device is touched: a bad config is reported as such on any machine
	if (rc != XALM_OK) { delete m; return rc; }
	int ndev = 0;
	cudaError_t e = cudaGetDeviceCount(&ndev);
	if (e != cudaSuccess) { delete m; return set_error(XALM_ERR_CUDA, "cudaGetDeviceCount failed: %s", cudaGetErrorString(e)); }
	if (device < 0 || device >= ndev) { delete m; return set_error(XALM_ERR_CUDA, "device %d not available (%d devices)", device, ndev); }
	e = cudaSetDevice(device);
	if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&m->own_stream, cudaStreamNonBlocking);
	if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&m->side, cudaStreamNonBlocking);
	if (e == cudaSuccess) e = cudaEventCreateWithFlags(&m->ev_fork, cudaEventDisableTiming);
	if (e == cudaSuccess) e = cudaEventCreateWithFlags(&m->ev_join, cudaEventDisableTiming);
	if (e != cudaSuccess) { delete m; return set_error(XALM_ERR_CUDA, "cudaStreamCreate failed: %s", cudaGetErrorString(e)); }
	m->stream = m->own_stream;
	*out = m;
	return XALM_OK;
}

int nb_upload(Nb* m, const char* name, int type_id, const int* shape, int rank, const void* data, size_t nbytes) {
	if (!m || !name || !shape || !data) return set_error(XALM_ERR_INVALID, "NULL argument");
	if (m->finalized) return set_error(XALM_ERR_STATE, "upload after finalize");
	auto it = m->tensors.find(name);
	if (it == m->tensors.end()) return set_error(XALM_ERR_INVALID, "unknown tensor name '%s'", name);
	HostTensor& t = it->second;
	bool same = (size_t) rank == t.shape.size();
	size_t count = 1;
	for (int i = 0; same && i < rank; i++) same = shape[i] == t.shape[(size_t) i];
	for (int dsz : t.shape) count *= (size_t) dsz;
	if (!same) return set_error(XALM_ERR_INVALID, "shape mismatch for %s", name);
	const size_t esz = type_id == XALM_F32 ? 4 : (type_id == XALM_F16 || type_id == XALM_BF16) ? 2 : 0;
	if (!esz) return set_error(XALM_ERR_UNSUPPORTED, "tensor %s: type %d (F32, F16 or BF16)", name, type_id);
	if (nbytes != count * esz) return set_error(XALM_ERR_INVALID, "size mismatch for %s", name);
	t.v.resize(count);
	if (type_id == XALM_F32) memcpy(t.v.data(), data, nbytes);
	else if (type_id == XALM_BF16) {
		const uint16_t* b = static_cast<const uint16_t*>(data);
		for (size_t i = 0; i < count; i++) {
			const uint32_t u = (uint32_t) b[i] << 16;
			memcpy(&t.v[i], &u, 4);
		}
	} else {
		const __half* hsrc = static_cast<const __half*>(data);
		for (size_t i = 0; i < count; i++) t.v[i] = __half2float(hsrc[i]);
	}
	t.type = type_id;
	t.got = true;
	return XALM_OK;
}

int nb_finalize(Nb* m) {
	if (!m) return set_error(XALM_ERR_INVALID, "model is NULL");
	if (m->finalized) return XALM_OK;
	XALM_CUDA_CHECK(cudaSetDevice(m->device));
	m->w_bf16 = m->precision != XALM_PRECISION_F32;
	for (const auto& [name, t] : m->tensors) {
		if (t.required && !t.got) return set_error(XALM_ERR_STATE, "tensor %s was not uploaded", name.c_str());
		if (t.matrix && t.got && t.type != XALM_BF16) m->w_bf16 = false; // wider checkpoints keep their precision
	}
	const int W = m->width, S = m->S;
	m->chunk = std::max(8, std::min(tune("seq_chunk"), 4096));
	m->keep_layers = getenv("XALM_SEQ_KEEP_LAYERS") ? atoi(getenv("XALM_SEQ_KEEP_LAYERS")) : 0;
	auto T = [&](const std::string& n) -> const HostTensor* {
		const HostTensor& t = m->tensors.at(n);
		return t.got ? &t : nullptr;
	};
	XALM_TRY(upload_rows(m, {T("embed")}, W, false, &m->embed, nullptr));
	XALM_TRY(upload_rows(m, {T("head")}, W, false, &m->w_head, &m->m_head));
	XALM_TRY(upload_vec(m, "final.norm", &m->final_norm));
	size_t max_proj = 0, max_att = 0, max_ro = 0, max_ff = 1, max_hdv = 0, max_h = 1;
	int max_ring = 1;
	for (size_t li = 0; li < m->layers.size(); li++) {
		Layer& L = m->layers[li];
		const std::string p = "l" + std::to_string(li) + ".";
		const int H = L.L.H, G = L.L.G, d = L.L.d, dv = L.L.dv, Hr = L.R.H, dr = L.R.d, dvr = L.R.dv;
		L.has_gate = T(p + "mix.left.g") != nullptr;
		L.off_lq = 0;
		L.off_lg = H * d;
		L.off_rq = L.off_lg + (L.has_gate ? H * dv : 0);
		L.off_rf = L.off_rq + Hr * dr;
		L.off_rv = L.off_rf + Hr * dr;
		L.n_plain = L.off_rv + Hr * dvr;
		L.n_in = L.n_plain + G * d + G * dv;
		XALM_TRY(upload_rows(m, {T(p + "mix.left.q"), T(p + "mix.left.g"), T(p + "mix.right.q"), T(p + "mix.right.f"), T(p + "mix.right.v"),
		                         T(p + "mix.left.k"), T(p + "mix.left.v")}, W, false, &L.w_in, &L.m_in));
		XALM_TRY(upload_rows(m, {T(p + "mix.left.o")}, H * dv, false, &L.w_lo, &L.m_lo));
		XALM_TRY(upload_rows(m, {T(p + "mix.right.o")}, Hr * dvr, false, &L.w_ro, &L.m_ro));
		if (L.has_mlp) {
			XALM_TRY(upload_rows(m, {T(p + "mlp.gate"), T(p + "mlp.up")}, W, true, &L.w_gu, &L.m_gu));
			XALM_TRY(upload_rows(m, {T(p + "mlp.down")}, L.ff, false, &L.w_down, &L.m_down));
			XALM_TRY(upload_vec(m, p + "norm2", &L.norm2));
			XALM_TRY(upload_vec(m, p + "ls2", &L.ls2));
		}
		XALM_TRY(upload_vec(m, p + "norm1", &L.norm1));
		XALM_TRY(upload_vec(m, p + "mix.left.r1", &L.r1));
		XALM_TRY(upload_vec(m, p + "mix.left.r2", &L.r2));
		if (!L.r1 != !L.r2) return set_error(XALM_ERR_STATE, "layer %zu: the distance bias needs both r1 and r2", li);
		XALM_TRY(upload_vec(m, p + "mix.left.talk", &L.talk));
		XALM_TRY(upload_vec(m, p + "mix.right.f.b", &L.fb));
		XALM_TRY(upload_vec(m, p + "mix.right.lower", &L.lower));
		XALM_TRY(upload_vec(m, p + "mix.right.norm", &L.rnorm));
		XALM_TRY(upload_vec(m, p + "mix.left.out", &L.lout));
		XALM_TRY(upload_vec(m, p + "mix.right.out", &L.rout));
		XALM_TRY(upload_vec(m, p + "ls1", &L.ls1));
		for (int q = 0; q < (L.has_mlp ? 2 : 1); q++) {
			const std::string hp = p + "hc" + std::to_string(q + 1) + ".";
			XALM_TRY(upload_vec(m, hp + "in", &L.hc_in[q]));
			XALM_TRY(upload_vec(m, hp + "out", &L.hc_out[q]));
			XALM_TRY(upload_vec(m, hp + "mix", &L.hc_mix[q]));
		}
		// the cache: a ring that holds one pass and the window before it
		const long long need = L.L.window > 0 ? (long long) L.L.window - 1 + m->chunk : (long long) m->max_tokens;
		L.ring = (int) std::min<long long>(need, m->max_tokens);
		const size_t kelem = m->precision == XALM_PRECISION_F32 ? 4 : 2;
		uint8_t *kc = nullptr, *vc = nullptr;
		XALM_TRY(dev_alloc(m, &kc, (size_t) L.ring * G * d * kelem, true));
		XALM_TRY(dev_alloc(m, &vc, (size_t) L.ring * G * dv * kelem, true));
		L.kc = kc; L.vc = vc;
		XALM_TRY(dev_alloc(m, &L.state, (size_t) Hr * dr * dvr, true));
		max_ring = std::max(max_ring, L.ring);
		max_proj = std::max(max_proj, (size_t) L.n_plain);
		max_att = std::max(max_att, (size_t) H * dv);
		max_ro = std::max(max_ro, (size_t) Hr * dvr);
		if (L.has_mlp) max_ff = std::max(max_ff, (size_t) L.ff);
		max_hdv = std::max(max_hdv, (size_t) H * dv);
		max_h = std::max(max_h, (size_t) H);
		const size_t asm_ = swa_smem_bytes(H, d, dv), hsm = hgrn2_smem_bytes(dr, dvr);
		if (!swa_pick_tq(H, G, d, dv, m->chunk) && asm_ > 200 * 1024)
			return set_error(XALM_ERR_UNSUPPORTED, "layer %zu: attention heads need %zu bytes of shared memory", li, asm_);
		if (!hgrn2_cols_ok(dr, dvr, m->chunk) && hsm > 200 * 1024)
			return set_error(XALM_ERR_UNSUPPORTED, "layer %zu: recurrence state needs %zu bytes of shared memory", li, hsm);
		XALM_TRY(swa_prepare(H, d, dv));
		XALM_TRY(hgrn2_prepare(dr, dvr));
	}
	XALM_TRY(hc_norm_prepare(W));
	// tensor-core operands: every matrix whose shape the GEMM takes keeps its fp16 tiles beside the bf16 rows the one-token steps stream
	m->use_tc = m->w_bf16 && tune("seq_tc") > 0;
	m->tc_min_rows = std::max(1, tune("seq_tc_min"));
	size_t a_bytes = 0, tc_cols = 4;
	if (m->use_tc) {
		auto build = [&](const WMat& wm, TcWeight* t) -> int {
			if (!tc_shape_ok(wm.rows, wm.n, wm.rows)) return XALM_OK; // this one stays on the fp32 kernels
			XALM_TRY(tc_weight_build(wm, 1, t, m->stream));
			a_bytes = std::max(a_bytes, tc_a_plane_bytes(m->chunk, wm.n));
			tc_cols = std::max(tc_cols, (size_t) wm.rows);
			m->weight_bytes_tc += (long long) t->NT * t->KT * 256 * 64 * 2;
			return XALM_OK;
		};
		for (Layer& L : m->layers) {
			XALM_TRY(build(L.m_in, &L.t_in));
			XALM_TRY(build(L.m_lo, &L.t_lo));
			XALM_TRY(build(L.m_ro, &L.t_ro));
			if (L.has_mlp) {
				XALM_TRY(build(L.m_gu, &L.t_gu));
				XALM_TRY(build(L.m_down, &L.t_down));
			}
		}
		XALM_TRY(build(m->m_head, &m->t_head));
		if (a_bytes) {
			XALM_TRY(dev_alloc(m, &m->a_hi, a_bytes, true));
			if (tune("seq_tc") >= 2) XALM_TRY(dev_alloc(m, &m->a_lo, a_bytes, true));
			XALM_TRY(dev_alloc(m, &m->tc_out, (size_t) m->chunk * tc_cols));
		} else m->use_tc = false;
		XALM_CUDA_CHECK(cudaStreamSynchronize(m->stream));
	}
	m->proj_ld = (max_proj + 3) / 4 * 4;
	const size_t C = (size_t) m->chunk;
	m->part_cap = std::max(4 * 64, 4 * m->chunk); // one-token steps: up to 64 key splits; passes of a prompt: up to 4 per token
	XALM_TRY(dev_alloc(m, &m->xs, (size_t) S * C * W));
	XALM_TRY(dev_alloc(m, &m->h, C * W));
	XALM_TRY(dev_alloc(m, &m->proj, C * m->proj_ld));
	XALM_TRY(dev_alloc(m, &m->att, C * max_att));
	XALM_TRY(dev_alloc(m, &m->ro, C * max_ro));
	XALM_TRY(dev_alloc(m, &m->ol, C * W));
	XALM_TRY(dev_alloc(m, &m->orr, C * W));
	XALM_TRY(dev_alloc(m, &m->y, C * max_ff));
	XALM_TRY(dev_alloc(m, &m->logits, C * m->vocab));
	XALM_TRY(dev_alloc(m, &m->part_o, (size_t) m->part_cap * max_hdv));
	XALM_TRY(dev_alloc(m, &m->part_ml, (size_t) m->part_cap * 2 * max_h));
	XALM_TRY(dev_alloc(m, &m->tickets, C, true));
	if (m->keep_layers) XALM_TRY(dev_alloc(m, &m->layer_sums, m->layers.size() * C * W, true));
	XALM_TRY(dev_alloc(m, &m->d_tokens, C));
	XALM_TRY(dev_alloc(m, &m->d_step, 1));
	XALM_CUDA_CHECK(cudaMallocHost(&m->h_logits, C * m->vocab * 4));
	for (auto& [name, t] : m->tensors) std::vector<float>().swap(t.v); // the device owns the weights from here on
	m->finalized = true;
	return XALM_OK;
}

int nb_release(Nb* m) {
	XALM_TRY(check_ready(m));
	XALM_CUDA_CHECK(cudaStreamSynchronize(m->stream));
	for (Layer& L : m->layers) XALM_CUDA_CHECK(cudaMemsetAsync(L.state, 0, (size_t) L.R.H * L.R.d * L.R.dv * 4, m->stream));
	XALM_CUDA_CHECK(cudaStreamSynchronize(m->stream));
	m->pos = 0;
	return XALM_OK;
}

int nb_forward(Nb* m, int token, int pos, int mode, float* logits_host) {
	return seq_step(m, &token, 1, pos, mode == XALM_OUTPUT_LOGITS ? 1 : 0, logits_host, nullptr, nullptr);
}
int nb_forward_async(Nb* m, int token, int pos, int mode) {
	XALM_TRY(check_ready(m));
	if (pos != m->pos) return set_error(XALM_ERR_STATE, "step: position %d, but the sequence holds %d tokens", pos, m->pos);
	if (pos + 1 > m->max_tokens) return set_error(XALM_ERR_INVALID, "step: position %d exceeds max_tokens %d", pos, m->max_tokens);
	return run_pass(m, &token, 1, mode == XALM_OUTPUT_LOGITS ? 1 : 0);
}
int nb_forward_argmax(Nb* m, int token, int pos, int* next) {
	if (!next) return set_error(XALM_ERR_INVALID, "next_token is NULL");
	XALM_TRY(seq_step(m, &token, 1, pos, 1, nullptr, nullptr, nullptr));
	int best = 0;
	for (int i = 1; i < m->vocab; i++)
		if (m->h_logits[i] > m->h_logits[best]) best = i;
	*next = best;
	return XALM_OK;
}
int nb_sync(Nb* m) {
	XALM_TRY(check_ready(m));
	XALM_CUDA_CHECK(cudaStreamSynchronize(m->stream));
	return XALM_OK;
}
int nb_prefill(Nb* m, const int* tokens, int n, int pos0, int want, float* logits_host, const int* targets, float* probs_host) {
	return seq_step(m, tokens, n, pos0, want, logits_host, targets, probs_host);
}
int nb_prefill_async(Nb* m, const int* tokens, int n, int pos0, int want) {
	XALM_TRY(check_ready(m));
	if (!tokens || n <= 0) return set_error(XALM_ERR_INVALID, "step: no tokens");
	if (pos0 != m->pos) return set_error(XALM_ERR_STATE, "step: position %d, but the sequence holds %d tokens", pos0, m->pos);
	if ((long long) pos0 + n > m->max_tokens) return set_error(XALM_ERR_INVALID, "step: positions exceed max_tokens %d", m->max_tokens);
	int total = 0;
	for (int at = 0; at < n; at += m->chunk) {
		const int nc = std::min(m->chunk, n - at);
		XALM_TRY(run_pass(m, tokens + at, nc, want == 2 ? 2 : (want == 1 && at + nc == n ? 1 : 0)));
		total += m->last_launches;
	}
	m->last_launches = total;
	return XALM_OK;
}
float* nb_logits_host(Nb* m) { return m ? m->h_logits : nullptr; }
int nb_set_stream(Nb* m, void* s) {
	if (!m) return set_error(XALM_ERR_INVALID, "model is NULL");
	m->stream = s ? (cudaStream_t) s : m->own_stream;
	return XALM_OK;
}
int nb_active_bytes(Nb* m, long long pos, long long* bytes) {
	if (!m || !bytes) return set_error(XALM_ERR_INVALID, "NULL argument");
	// what a one-token step at `pos` reads: every weight once (one embedding row), the visible K/V rows, the recurrent state twice
	long long b = m->weight_bytes - (long long) (m->vocab - 1) * m->width * (m->w_bf16 ? 2 : 4);
	const long long kelem = m->precision == XALM_PRECISION_F32 ? 4 : 2;
	for (const Layer& L : m->layers) {
		const long long seen = L.L.window > 0 ? std::min<long long>(pos + 1, L.L.window) : pos + 1;
		b += seen * L.L.G * (L.L.d + L.L.dv) * kelem + 2ll * L.R.H * L.R.d * L.R.dv * 4;
	}
	*bytes = b;
	return XALM_OK;
}
int nb_last_launch_count(Nb* m, int* n) {
	if (!m || !n) return set_error(XALM_ERR_INVALID, "NULL argument");
	*n = m->last_launches;
	return XALM_OK;
}
// which: XALM_S_LOGITS = logits of the last pass (rows x vocab); 100 + l = the residual stream (sum of the streams) after layer l for the
// rows of the last pass (kept only when XALM_SEQ_KEEP_LAYERS=1 was set at finalize); 1000 + l = recurrent state of layer l
int nb_read_state(Nb* m, int which, float* dst, size_t n) {
	XALM_TRY(check_ready(m));
	if (!dst) return set_error(XALM_ERR_INVALID, "dst is NULL");
	XALM_CUDA_CHECK(cudaStreamSynchronize(m->stream));
	const float* src = nullptr;
	size_t cap = 0;
	if (which == XALM_S_LOGITS) { src = m->logits; cap = (size_t) m->chunk * m->vocab; }
	else if (which >= 100 && which < 100 + (int) m->layers.size() && m->layer_sums) {
		src = m->layer_sums + (size_t) (which - 100) * m->chunk * m->width;
		cap = (size_t) m->chunk * m->width;
	} else if (which >= 1000 && which < 1000 + (int) m->layers.size()) {
		const Layer& L = m->layers[(size_t) (which - 1000)];
		src = L.state;
		cap = (size_t) L.R.H * L.R.d * L.R.dv;
	} else return set_error(XALM_ERR_INVALID, "read_state: buffer %d", which);
	if (n > cap) return set_error(XALM_ERR_INVALID, "read_state: %zu elements requested, buffer holds %zu", n, cap);
	XALM_CUDA_CHECK(cudaMemcpy(dst, src, n * 4, cudaMemcpyDeviceToHost));
	return XALM_OK;
}
int nb_expected_tensor(Nb* m, int index, char* name, size_t cap, int* shape4, int* rank) {
	if (!m || !name || !shape4 || !rank) return set_error(XALM_ERR_INVALID, "NULL argument");
	if (index < 0 || index >= (int) m->order.size()) return set_error(XALM_ERR_INVALID, "no tensor %d", index);
	const std::string& nm = m->order[(size_t) index];
	const HostTensor& t = m->tensors.at(nm);
	snprintf(name, cap, "%s", nm.c_str());
	*rank = (int) t.shape.size();
	for (size_t i = 0; i < t.shape.size() && i < 4; i++) shape4[i] = t.shape[i];
	return XALM_OK;
}
int nb_info(Nb* m, const char* key, long long* value) {
	if (!m || !key || !value) return set_error(XALM_ERR_INVALID, "NULL argument");
	const std::string k = key;
	if (k == "vocab_size") *value = m->vocab;
	else if (k == "dim") *value = m->width;
	else if (k == "n_layers") *value = (long long) m->layers.size();
	else if (k == "max_tokens") *value = m->max_tokens;
	else if (k == "position") *value = m->pos;
	else if (k == "chunk") *value = m->chunk;
	else return set_error(XALM_ERR_INVALID, "unknown property '%s'", key);
	return XALM_OK;
}

// the family table speaks in opaque handles
template <auto F>
struct Thunk;
template <typename... A, int (*F)(Nb*, A...)>
struct Thunk<F> {
	static int call(xalm_cuda_model* h, A... a) { return F(reinterpret_cast<Nb*>(h), a...); }
};
int create_thunk(const char* json, int device, int max_tokens, int precision, xalm_cuda_model** out) {
	return nb_create(json, device, max_tokens, precision, reinterpret_cast<Nb**>(out));
}
void destroy_thunk(xalm_cuda_model* h) { nb_destroy(reinterpret_cast<Nb*>(h)); }
float* logits_thunk(xalm_cuda_model* h) { return nb_logits_host(reinterpret_cast<Nb*>(h)); }

const ModelFamily nabalix_family = {
    "Nabalix", create_thunk, Thunk<nb_upload>::call, nullptr, nullptr, Thunk<nb_finalize>::call, destroy_thunk, nullptr, nullptr, nullptr,
    Thunk<nb_set_stream>::call, Thunk<nb_forward>::call, Thunk<nb_forward_argmax>::call, Thunk<nb_forward_async>::call, Thunk<nb_sync>::call,
    Thunk<nb_prefill>::call, Thunk<nb_prefill_async>::call, logits_thunk, Thunk<nb_active_bytes>::call, Thunk<nb_last_launch_count>::call,
    Thunk<nb_read_state>::call, nullptr, nullptr, Thunk<nb_release>::call, Thunk<nb_expected_tensor>::call, Thunk<nb_info>::call, nullptr};
const FamilyRegistrar nabalix_registrar(&nabalix_family);

} // namespace
} // namespace xalm
