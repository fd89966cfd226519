// nabalix.cu — the Nabalix family of the model registry (family.h): a decoder-only model described by a config.json whose
// layers run two token mixers side by side on the same normed input — windowed softmax attention (grouped K/V heads, soft-capped
// scores, logarithmic distance bias, score mixing across heads, sigmoid output gate) and an HGRN2 gated linear recurrence — join
// them as the mean of their RMS-normed outputs, follow with a clamped-GLU feed-forward, and carry the residual in several
// hyper-connected streams with a layer scale on every sublayer.
//
// The step function, the graph of one-token steps, tensor upload and the entry points are the shared sequence engine's
// (seq_family.cuh); this file holds what is Nabalix: its configuration, device layouts, cache and state, and the kernels of a pass.
// Per pass and layer:
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
#include "seq_family.cuh"

namespace xalm {
namespace {

using namespace mix;
using namespace seq;

struct LeftCfg {
	int H = 0, G = 0, d = 0, dv = 0, window = 0; // window 0: every earlier position is visible
	float scale = 1.f, softcap = 0.f;
};
struct RightCfg {
	int H = 0, d = 0, dv = 0;
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

struct NabalixModel : SeqModel {
	int S = 1;
	std::vector<Layer> layers;
	// activations of one pass
	float *xs = nullptr, *h = nullptr, *proj = nullptr, *att = nullptr, *ro = nullptr, *ol = nullptr, *orr = nullptr, *y = nullptr;
	float *part_o = nullptr, *part_ml = nullptr;
	unsigned* tickets = nullptr; // per query tile: arrivals of the attention's key splits
	int part_cap = 0;            // (token, key split) pairs the attention's partial buffers hold
	size_t proj_ld = 0;
};
typedef NabalixModel Nb;

// ---- config.json ------------------------------------------------------------------------------------------------------------
int parse_config(SeqModel* sm, const char* json) {
	Nb* m = static_cast<Nb*>(sm);
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
		m->n_layers = (int) m->layers.size();
		expect(m, "final.norm", {W}, false);
		expect(m, "head", {m->vocab, W}, true);
	} catch (const std::exception& e) {
		return set_error(XALM_ERR_INVALID, "config.json: %s", e.what());
	}
	return XALM_OK;
}

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
int enqueue_pass(SeqModel* sm, int n, int want, int* nl) {
	Nb* m = static_cast<Nb*>(sm);
	cudaStream_t s = m->stream;
	const int W = m->width, S = m->S;
	const size_t sstride = (size_t) m->chunk * W;
	const int rt = norm_threads(W);
	if (m->w_bf16) embed_streams_kernel<__nv_bfloat16><<<n, rt, 0, s>>>((const __nv_bfloat16*) m->embed, m->d_tokens, W, S, sstride, m->xs);
	else embed_streams_kernel<float><<<n, rt, 0, s>>>((const float*) m->embed, m->d_tokens, W, S, sstride, m->xs);
	XALM_SEQ_LAUNCH_CHECK("embed");
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

// ---- device layouts, cache, state, pass buffers ---------------------------------------------------------------------------------
int finalize(SeqModel* sm) {
	Nb* m = static_cast<Nb*>(sm);
	const int W = m->width, S = m->S;
	auto T = [&](const std::string& n) { return tensor_or_null(m, n); };
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
	for (Layer& L : m->layers) {
		XALM_TRY(tc_register(m, L.m_in, &L.t_in));
		XALM_TRY(tc_register(m, L.m_lo, &L.t_lo));
		XALM_TRY(tc_register(m, L.m_ro, &L.t_ro));
		if (L.has_mlp) {
			XALM_TRY(tc_register(m, L.m_gu, &L.t_gu));
			XALM_TRY(tc_register(m, L.m_down, &L.t_down));
		}
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
	(void) max_ring;
	return XALM_OK;
}

int release(SeqModel* sm) {
	Nb* m = static_cast<Nb*>(sm);
	for (Layer& L : m->layers) XALM_CUDA_CHECK(cudaMemsetAsync(L.state, 0, (size_t) L.R.H * L.R.d * L.R.dv * 4, m->stream));
	return XALM_OK;
}

// beyond the matrices: the visible K/V rows, the recurrent state twice
long long active_bytes(SeqModel* sm, long long pos) {
	Nb* m = static_cast<Nb*>(sm);
	long long b = 0;
	const long long kelem = m->precision == XALM_PRECISION_F32 ? 4 : 2;
	for (const Layer& L : m->layers) {
		const long long seen = L.L.window > 0 ? std::min<long long>(pos + 1, L.L.window) : pos + 1;
		b += seen * L.L.G * (L.L.d + L.L.dv) * kelem + 2ll * L.R.H * L.R.d * L.R.dv * 4;
	}
	return b;
}

bool state_buffer(SeqModel* sm, int layer, const float** src, size_t* count) {
	Nb* m = static_cast<Nb*>(sm);
	const Layer& L = m->layers[(size_t) layer];
	*src = L.state;
	*count = (size_t) L.R.H * L.R.d * L.R.dv;
	return true;
}

void destroy(SeqModel* sm) {
	Nb* m = static_cast<Nb*>(sm);
	for (Layer& L : m->layers)
		for (TcWeight* t : {&L.t_in, &L.t_lo, &L.t_ro, &L.t_gu, &L.t_down}) tc_weight_free(t);
	delete m;
}

const SeqHooks nabalix_hooks = {parse_config, finalize, enqueue_pass, release, active_bytes, state_buffer, destroy};
extern const ModelFamily nabalix_family;
int create(const char* json, int device, int max_tokens, int precision, xalm_cuda_model** out) {
	return seq_create<Nb>(&nabalix_family, &nabalix_hooks, json, device, max_tokens, precision, out);
}
const ModelFamily nabalix_family = seq_family_table("Nabalix", create);
const FamilyRegistrar nabalix_registrar(&nabalix_family);

} // namespace
} // namespace xalm
