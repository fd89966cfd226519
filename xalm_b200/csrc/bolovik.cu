// bolovik.cu — the Bolovik family of the model registry (family.h): a decoder-only model described by a config.json whose layers
// each carry ONE token mixer, chosen per layer, and an optional feed-forward:
//
//   mixer "attention"  softmax attention with grouped K/V heads, biases on q / k / v, rotary positions on part of each head (rotate-half
//                      pairs, frequencies rescaled by wavelength bands), weightless RMS norms of q, k (after rotation) and v, a sliding
//                      window that also keeps the sequence's first positions visible
//   mixer "delta"      gated delta rule: short causal convolutions + silu on q / k / v, unit-length q and k, per-head decay and write
//                      strength, fp32 state, per-head RMS norm and silu output gate
//   feed-forward       dense gated (tanh-gelu) or a mixture of small silu-gated experts: sigmoid router scores, expert groups limiting
//                      the choice, weights = the chosen scores
//
// Sublayers read the residual stream as it is and are normed on the way OUT: x <- x + gnorm(sublayer(x)) with an RMS norm taken over
// `norm.groups` equal parts of the row.  What a layer hands on is a learned average over the depth: sum_j dwa[j] X_j of the embedding
// output X_0 and every layer result so far.
//
// The step function, graph replay of one-token steps, uploads, release and the C entry points are the shared sequence engine's
// (seq_family.cuh).  Per pass and layer here:
//     attention: rows product [q | k | v]  ->  qkv_post (bias, rotation, norms, cache write)  ->  swa_attn / swa_tile (window + kept
//                first positions)  ->  rows product [o]  ->  group_norm_residual
//     delta:     rows product [q | k | v | gate | b | a]  ->  delta_prep  ->  delta_rule  ->  rows product [o]  ->  group_norm_residual
//     dense ff:  rows product [gate | up interleaved, gelu GLU fused]  ->  rows product [down]  ->  group_norm_residual (+ depth average)
//     experts:   moe_router  ->  moe_sort  ->  moe_gemm [gate | up, silu GLU fused]  ->  moe_gemm [down]  ->  group_norm_residual, which
//                sums the chosen experts' rows with their weights (+ depth average)
//
// Cache / state manager: an attention layer keeps keep_first pinned slots and a ring of min(max_tokens, window - 1 + seq_chunk) slots
// behind them (position p >= keep_first lives in slot keep_first + (p - keep_first) mod ring); a delta layer keeps its fp32 state
// (heads x dim x vdim) and the last taps - 1 inputs of every convolved channel.  release() zeroes the delta layers' state; cache slots
// need no clearing, a sequence only reads positions it has written.
//
// Precision: the residual stream, norms, rotation angles, scores, softmax, router, gates, decays and the recurrence are fp32 in both
// modes.  XALM_PRECISION_BF16 keeps matrices and the K/V cache in bf16 and sends dense products of long passes through the tcgen05 GEMM
// (fp16 operands, fp32 accumulation); XALM_PRECISION_F32 widens both and uses the fp32 FMA kernels only.
#include "seq_family.cuh"

#include "delta_ops.cuh"
#include "moe_ops.cuh"

namespace xalm {
namespace {

using namespace mix;
using namespace seq;

enum { MIX_ATTENTION = 0, MIX_DELTA = 1 };
enum { FF_NONE = 0, FF_DENSE = 1, FF_MOE = 2 };

struct Layer {
	int mixer = MIX_ATTENTION, ff_kind = FF_NONE;
	int H = 0, G = 0, d = 0, dv = 0;
	// attention
	int window = 0x7fffffff, keep_first = 0, rot_dims = 0;
	float scale = 1.f;
	std::vector<float> freq_host;
	float *freq = nullptr, *bq = nullptr, *bk = nullptr, *bv = nullptr;
	void *kc = nullptr, *vc = nullptr;
	int ring = 1;
	// delta
	int taps = 1;
	float *cq = nullptr, *ck = nullptr, *cv = nullptr, *A_log = nullptr, *dt_bias = nullptr, *onorm = nullptr;
	float *state = nullptr, *conv_state = nullptr;
	int off_k = 0, off_v = 0, off_g = 0, off_b = 0, off_a = 0, n_in = 0;
	// feed-forward
	int ff = 0, E = 0, top = 0, n_groups = 0, keep_groups = 0;
	// device
	void *w_in = nullptr, *w_o = nullptr, *w_gu = nullptr, *w_down = nullptr, *w_router = nullptr;
	WMat m_in, m_o, m_gu, m_down;
	TcWeight t_in, t_o, t_gu, t_down;
	std::vector<TcWeight> t_egu, t_edown; // per expert, when the mixture's long passes run on the tensor cores
	float *norm1 = nullptr, *norm2 = nullptr, *dwa = nullptr;
};

struct BolovikModel : SeqModel {
	int groups = 1;
	std::vector<Layer> layers;
	// one pass
	float *hist = nullptr, *xavg = nullptr; // results X_0 .. X_L of the pass's rows; what the next layer reads
	float *proj = nullptr, *prep = nullptr, *att = nullptr, *y = nullptr, *ffh = nullptr, *hn = nullptr;
	int proj_ld = 4, prep_ld = 4;
	float *part_o = nullptr, *part_ml = nullptr;
	unsigned* tickets = nullptr;
	int part_cap = 0;
	int *moe_idx = nullptr, *moe_sorted = nullptr, *moe_tiles = nullptr, *moe_ntiles = nullptr;
	float *moe_wgt = nullptr, *moe_hid = nullptr, *moe_out = nullptr;
	int *moe_off = nullptr, *moe_inv = nullptr, *h_off = nullptr; // first place of every expert in the sorted pairs (device, pinned host), inverse order
	float* moe_x = nullptr;                                        // the pairs' input rows in sorted order
};
typedef BolovikModel Bv;

// ---- config.json ------------------------------------------------------------------------------------------------------------------
// rotary frequencies f_i = base^(-2i/dims), rescaled by wavelength l = 2 pi / f: kept where l < original / high, divided by `factor` where
// l > original / low, blended linearly in (original / l) between the two
std::vector<float> rotary_frequencies(const xjson::Value& rot, int dims) {
	const double base = getf(rot, "base");
	const xjson::Value* sc = rot.find("scaling");
	const bool scaled = sc && sc->kind == xjson::Value::Obj;
	double factor = 1, low = 1, high = 1, original = 1;
	if (scaled) { factor = getf(*sc, "factor"); low = getf(*sc, "low"); high = getf(*sc, "high"); original = getf(*sc, "original"); }
	std::vector<float> f((size_t) dims / 2);
	for (int i = 0; i < dims / 2; i++) {
		double fi = pow(base, -2.0 * i / dims);
		if (scaled) {
			const double l = 2.0 * M_PI / fi;
			if (l > original / low) fi /= factor;
			else if (l >= original / high) {
				const double s = (original / l - low) / (high - low);
				fi = (1.0 - s) * fi / factor + s * fi;
			}
		}
		f[(size_t) i] = (float) fi;
	}
	return f;
}

int parse_config(SeqModel* sm, const char* json) {
	Bv* m = static_cast<Bv*>(sm);
	try {
		const xjson::Value c = xjson::Parser::parse(json, strlen(json));
		m->vocab = geti(c, "vocab");
		m->width = geti(c, "width");
		if (const xjson::Value* nv = c.find("norm")) {
			if (const xjson::Value* e = nv->find("eps")) m->eps = (float) e->num;
			if (nv->contains("groups")) m->groups = geti(*nv, "groups");
		}
		if (m->vocab <= 0 || m->width <= 0) return set_error(XALM_ERR_INVALID, "config: vocab / width must be positive");
		if (m->groups <= 0 || m->width % m->groups) return set_error(XALM_ERR_INVALID, "config: %d norm groups do not divide the width %d", m->groups, m->width);
		const int W = m->width;
		expect(m, "embed", {m->vocab, W}, true);
		const xjson::Value& layers = c.at("layers");
		if (layers.kind != xjson::Value::Array || layers.arr.empty()) return set_error(XALM_ERR_INVALID, "config: no layers");
		for (size_t li = 0; li < layers.arr.size(); li++) {
			const xjson::Value& lv = layers.arr[li];
			const std::string type = lv.at("type").str;
			Layer L;
			if (type == "attention") L.mixer = MIX_ATTENTION;
			else if (type == "delta") L.mixer = MIX_DELTA;
			else return set_error(XALM_ERR_UNSUPPORTED, "config: layer %zu has mixer type '%s' (this family runs 'attention' and 'delta')", li, type.c_str());
			const xjson::Value& mx = lv.at("mixer");
			L.H = geti(mx, "heads");
			L.G = mx.contains("kv_heads") ? geti(mx, "kv_heads") : L.H;
			L.d = geti(mx, "dim");
			L.dv = mx.contains("vdim") ? geti(mx, "vdim") : L.d;
			if (L.H <= 0 || L.G <= 0 || L.H % L.G || L.d <= 0 || L.dv <= 0) return set_error(XALM_ERR_INVALID, "config: layer %zu: bad mixer sizes", li);
			const std::string p = "l" + std::to_string(li) + ".";
			const int H = L.H, G = L.G, d = L.d, dv = L.dv;
			expect(m, p + "norm1", {W}, false);
			if (L.mixer == MIX_ATTENTION) {
				L.scale = mx.contains("scale") ? (float) getf(mx, "scale") : 1.f / sqrtf((float) d);
				if (const xjson::Value* mk = mx.find("mask"); mk && mk->kind == xjson::Value::Obj) {
					if (mk->contains("size")) L.window = geti(*mk, "size");
					if (mk->contains("keep_first")) L.keep_first = geti(*mk, "keep_first");
					if (L.window <= 0 || L.keep_first < 0) return set_error(XALM_ERR_INVALID, "config: layer %zu: bad mask", li);
					if (L.window == 0x7fffffff) L.keep_first = 0; // no window: everything is visible anyway
				}
				if (const xjson::Value* rt = mx.find("rot"); rt && rt->kind == xjson::Value::Obj) {
					L.rot_dims = geti(*rt, "dims");
					if (L.rot_dims < 0 || L.rot_dims > d || L.rot_dims % 2) return set_error(XALM_ERR_INVALID, "config: layer %zu: %d rotary dimensions in a head of %d", li, L.rot_dims, d);
					if (L.rot_dims) L.freq_host = rotary_frequencies(*rt, L.rot_dims);
				}
				expect(m, p + "mix.q", {H * d, W}, true);
				expect(m, p + "mix.q.b", {H * d}, false, false);
				expect(m, p + "mix.k", {G * d, W}, true);
				expect(m, p + "mix.k.b", {G * d}, false, false);
				expect(m, p + "mix.v", {G * dv, W}, true);
				expect(m, p + "mix.v.b", {G * dv}, false, false);
				expect(m, p + "mix.o", {W, H * dv}, true);
			} else {
				L.taps = mx.contains("conv") ? geti(mx, "conv") : 1;
				if (L.taps < 1) return set_error(XALM_ERR_INVALID, "config: layer %zu: conv", li);
				if (!delta_ok(d, dv)) return set_error(XALM_ERR_UNSUPPORTED, "config: layer %zu: a delta-rule state of %d x %d per head", li, d, dv);
				expect(m, p + "mix.q", {G * d, W}, true);
				expect(m, p + "mix.q.conv", {G * d, L.taps}, false);
				expect(m, p + "mix.k", {G * d, W}, true);
				expect(m, p + "mix.k.conv", {G * d, L.taps}, false);
				expect(m, p + "mix.v", {H * dv, W}, true);
				expect(m, p + "mix.v.conv", {H * dv, L.taps}, false);
				expect(m, p + "mix.b", {H, W}, true);
				expect(m, p + "mix.A_log", {H}, false);
				expect(m, p + "mix.norm", {dv}, false);
				expect(m, p + "mix.a", {H, W}, true);
				expect(m, p + "mix.dt_bias", {H}, false);
				expect(m, p + "mix.g", {H * dv, W}, true);
				expect(m, p + "mix.o", {W, H * dv}, true);
			}
			const xjson::Value* mlp = lv.find("mlp");
			if (mlp && mlp->kind == xjson::Value::Obj) {
				const std::string kind = mlp->contains("kind") ? mlp->at("kind").str : "dense";
				expect(m, p + "norm2", {W}, false);
				if (kind == "dense") {
					L.ff_kind = FF_DENSE;
					L.ff = geti(*mlp, "ff");
					if (L.ff <= 0) return set_error(XALM_ERR_INVALID, "config: layer %zu: ff", li);
					expect(m, p + "mlp.gate", {L.ff, W}, true);
					expect(m, p + "mlp.up", {L.ff, W}, true);
					expect(m, p + "mlp.down", {W, L.ff}, true);
				} else if (kind == "moe") {
					L.ff_kind = FF_MOE;
					L.ff = geti(mlp->at("expert"), "ff");
					const xjson::Value& r = mlp->at("router");
					L.E = geti(r, "experts");
					L.top = geti(r, "top");
					if (const xjson::Value* g = r.find("groups"); g && g->kind == xjson::Value::Obj) {
						L.n_groups = geti(*g, "count");
						L.keep_groups = geti(*g, "keep");
					}
					if (L.ff <= 0 || L.E <= 0 || L.top <= 0 || L.top > L.E) return set_error(XALM_ERR_INVALID, "config: layer %zu: %d of %d experts of %d", li, L.top, L.E, L.ff);
					if (L.n_groups > 1 && (L.E % L.n_groups || L.keep_groups <= 0 || L.keep_groups > L.n_groups || L.keep_groups * (L.E / L.n_groups) < L.top))
						return set_error(XALM_ERR_INVALID, "config: layer %zu: %d expert groups with %d kept cannot hold %d of %d experts", li, L.n_groups, L.keep_groups, L.top, L.E);
					for (int e = 0; e < L.E; e++) {
						const std::string pe = p + "mlp.e" + std::to_string(e) + ".";
						expect(m, pe + "gate", {L.ff, W}, true);
						expect(m, pe + "up", {L.ff, W}, true);
						expect(m, pe + "down", {W, L.ff}, true);
					}
					expect(m, p + "mlp.router", {L.E, W}, true);
				} else return set_error(XALM_ERR_UNSUPPORTED, "config: layer %zu has feed-forward kind '%s'", li, kind.c_str());
			}
			expect(m, p + "dwa", {(int) li + 2}, false, false);
			m->layers.push_back(std::move(L));
		}
		m->n_layers = (int) m->layers.size();
		expect(m, "final.norm", {W}, false);
		expect(m, "head", {m->vocab, W}, true);
	} catch (const std::exception& e) {
		return set_error(XALM_ERR_INVALID, "config.json: %s", e.what());
	}
	return XALM_OK;
}

// ---- the kernels of one pass ----------------------------------------------------------------------------------------------------------
// x + gnorm(y) for one sublayer; with `last` the layer's result lands in hist[li + 1] and the depth average (if the layer has one) in xavg
int enqueue_norm_add(Bv* m, size_t li, const Layer& L, bool second, bool last, const float* x_in, const float* y, int ldy, int parts, const float* part_w,
                     const int* part_row, int n, int* nl) {
	const size_t hs = (size_t) m->chunk * m->width;
	GroupNormArgs g;
	g.y = y; g.ldy = ldy; g.parts = parts; g.part_w = part_w; g.part_row = part_row;
	g.w = second ? L.norm2 : L.norm1;
	g.groups = m->groups; g.width = m->width; g.eps = m->eps;
	g.x_in = x_in;
	g.x_out = m->hist + (li + 1) * hs;
	if (last) {
		if (L.dwa) {
			g.hist = m->hist; g.hist_stride = hs; g.n_hist = (int) li + 1; g.dwa = L.dwa; g.avg_out = m->xavg;
		}
		if (m->keep_layers) g.keep_out = m->layer_sums + li * hs;
	}
	XALM_TRY(launch_group_norm(g, n, m->stream));
	(*nl)++;
	return XALM_OK;
}

int enqueue_pass(SeqModel* sm, int n, int want, int* nl) {
	Bv* m = static_cast<Bv*>(sm);
	cudaStream_t s = m->stream;
	const int W = m->width;
	const size_t hs = (size_t) m->chunk * W;
	const bool f32 = m->precision == XALM_PRECISION_F32;
	if (m->w_bf16) embed_streams_kernel<__nv_bfloat16><<<n, norm_threads(W), 0, s>>>((const __nv_bfloat16*) m->embed, m->d_tokens, W, 1, hs, m->hist);
	else embed_streams_kernel<float><<<n, norm_threads(W), 0, s>>>((const float*) m->embed, m->d_tokens, W, 1, hs, m->hist);
	XALM_SEQ_LAUNCH_CHECK("embed");
	const float* x = m->hist; // what the layer reads: X_0, later the depth average (or the last result where a layer has none)
	for (size_t li = 0; li < m->layers.size(); li++) {
		const Layer& L = m->layers[li];
		const int H = L.H, G = L.G, d = L.d, dv = L.dv;
		RowsEpi est;
		est.kind = EPI_STORE; est.out = m->proj; est.ldo = m->proj_ld;
		XALM_TRY(rows_product(m, x, W, L.w_in, &L.t_in, n, L.n_in, W, est, nl));
		if (L.mixer == MIX_ATTENTION) {
			QkvPostArgs qa = {};
			qa.proj = m->proj; qa.ld = m->proj_ld; qa.q_off = 0; qa.k_off = H * d; qa.v_off = H * d + G * d;
			qa.H = H; qa.G = G; qa.d = d; qa.dv = dv;
			qa.bq = L.bq; qa.bk = L.bk; qa.bv = L.bv;
			qa.freq = L.freq; qa.rot_half = L.rot_dims / 2;
			qa.norm_qk = 1; qa.norm_v = 1; qa.eps = m->eps;
			qa.kc = L.kc; qa.vc = L.vc; qa.cache_f32 = f32; qa.keep_first = L.keep_first; qa.ring = L.ring;
			qa.step = m->d_step;
			XALM_TRY(launch_qkv_post(qa, n, s));
			(*nl)++;
			SwaArgs sa = {};
			sa.q = m->proj; sa.ldq = m->proj_ld; sa.q_off = 0;
			sa.kc = L.kc; sa.vc = L.vc; sa.ring = L.ring; sa.keep_first = L.keep_first;
			sa.H = H; sa.G = G; sa.d = d; sa.dv = dv;
			sa.window = L.window; sa.scale = L.scale;
			sa.step = m->d_step; sa.out = m->att;
			sa.n_splits = 0;
			sa.part_o = m->part_o; sa.part_ml = m->part_ml; sa.part_cap = m->part_cap; sa.tickets = m->tickets;
			int swa_launches = 1;
			XALM_TRY(launch_swa(sa, n, f32, s, &swa_launches));
			*nl += swa_launches;
		} else {
			DeltaArgs da = {};
			da.proj = m->proj; da.ld = m->proj_ld;
			da.q_off = 0; da.k_off = L.off_k; da.v_off = L.off_v; da.g_off = L.off_g; da.b_off = L.off_b; da.a_off = L.off_a;
			da.H = H; da.G = G; da.d = d; da.dv = dv; da.taps = L.taps;
			da.wq = L.cq; da.wk = L.ck; da.wv = L.cv; da.A_log = L.A_log; da.dt_bias = L.dt_bias; da.norm_w = L.onorm;
			da.eps = m->eps; da.unit_eps = 1e-6f; da.q_scale = 1.f / sqrtf((float) d);
			da.conv_state = L.conv_state; da.state = L.state;
			da.prep = m->prep; da.ldp = m->prep_ld; da.out = m->att; da.step = m->d_step;
			XALM_TRY(launch_delta(da, n, s));
			*nl += 2;
		}
		est.out = m->y; est.ldo = W;
		XALM_TRY(rows_product(m, m->att, H * dv, L.w_o, &L.t_o, n, W, H * dv, est, nl));
		XALM_TRY(enqueue_norm_add(m, li, L, false, L.ff_kind == FF_NONE, x, m->y, W, 1, nullptr, nullptr, n, nl));
		const float* x1 = m->hist + (li + 1) * hs;
		if (L.ff_kind == FF_DENSE) {
			RowsEpi eg;
			eg.kind = EPI_GLU; eg.glu_act = GLU_GELU_TANH; eg.out = m->ffh; eg.ldo = L.ff;
			XALM_TRY(rows_product(m, x1, W, L.w_gu, &L.t_gu, n, 2 * L.ff, W, eg, nl));
			est.out = m->y; est.ldo = W;
			XALM_TRY(rows_product(m, m->ffh, L.ff, L.w_down, &L.t_down, n, W, L.ff, est, nl));
			XALM_TRY(enqueue_norm_add(m, li, L, true, true, x1, m->y, W, 1, nullptr, nullptr, n, nl));
		} else if (L.ff_kind == FF_MOE) {
			MoeRouteArgs ra = {};
			ra.h = x1; ra.ldh = W; ra.w = L.w_router; ra.w_bf16 = m->w_bf16;
			ra.E = L.E; ra.top = L.top; ra.K = W; ra.n_groups = L.n_groups; ra.keep_groups = L.keep_groups;
			ra.idx = m->moe_idx; ra.wgt = m->moe_wgt; ra.step = m->d_step;
			XALM_TRY(launch_moe_router(ra, n, s));
			const bool on_tc = m->use_tc && !L.t_egu.empty() && n >= m->tc_min_rows;
			const bool tiled = on_tc || n * L.top > MOE_MATVEC_PAIRS; // steps of a few tokens run one matvec per (token, slot) pair and need no tile list
			if (tiled) {
				MoeSortArgs so = {m->moe_idx, L.top, L.E, m->d_step, m->moe_sorted, m->moe_tiles, m->moe_ntiles, m->moe_off, m->moe_inv};
				XALM_TRY(launch_moe_sort(so, s));
				(*nl)++;
			}
			(*nl)++;
			if (on_tc) {
				// Long passes of the 16-bit mode: each expert's rows, gathered one after the other, go through the tcgen05 GEMM on that expert's
				// resident fp16 tiles.  How many rows each expert got is read back first (one small copy and a wait per mixture layer and pass).
				XALM_CUDA_CHECK(cudaMemcpyAsync(m->h_off, m->moe_off, (size_t) (L.E + 1) * 4, cudaMemcpyDeviceToHost, s));
				moe_gather_kernel<<<n * L.top, 256, 0, s>>>(x1, W, L.top, m->moe_sorted, m->d_step, L.top, W, m->moe_x);
				XALM_SEQ_LAUNCH_CHECK("moe_gather");
				XALM_CUDA_CHECK(cudaStreamSynchronize(s));
				RowsEpi eg;
				eg.kind = EPI_GLU; eg.glu_act = GLU_SILU; eg.ldo = L.ff;
				for (int e = 0; e < L.E; e++) {
					const int at = m->h_off[e], cnt = m->h_off[e + 1] - at;
					if (cnt <= 0) continue;
					XALM_TRY(tc_gemm(L.t_egu[(size_t) e], m->moe_x + (size_t) at * W, cnt, m->tc_out, 2 * L.ff, m->a_hi, m->a_lo, s));
					eg.out = m->moe_hid + (size_t) at * L.ff;
					XALM_TRY(launch_rows_epilogue(m->tc_out, 2 * L.ff, cnt, 2 * L.ff, eg, s));
					XALM_TRY(tc_gemm(L.t_edown[(size_t) e], m->moe_hid + (size_t) at * L.ff, cnt, m->moe_out + (size_t) at * W, W, m->a_hi, m->a_lo, s));
					*nl += 5;
				}
			} else {
				MoeGemmArgs ga = {};
				ga.A = x1; ga.lda = W; ga.a_div = L.top; ga.W = L.w_gu; ga.N = 2 * L.ff; ga.K = W;
				ga.sorted = m->moe_sorted; ga.tiles = m->moe_tiles; ga.n_tiles = m->moe_ntiles;
				ga.idx = m->moe_idx; ga.step = m->d_step; ga.top = L.top;
				ga.e.kind = EPI_GLU; ga.e.glu_act = GLU_SILU; ga.e.out = m->moe_hid; ga.e.ldo = L.ff;
				XALM_TRY(launch_moe_gemm(ga, m->w_bf16, n * L.top, L.E, s));
				ga.A = m->moe_hid; ga.lda = L.ff; ga.a_div = 1; ga.W = L.w_down; ga.N = W; ga.K = L.ff;
				ga.e = RowsEpi();
				ga.e.kind = EPI_STORE; ga.e.out = m->moe_out; ga.e.ldo = W;
				XALM_TRY(launch_moe_gemm(ga, m->w_bf16, n * L.top, L.E, s));
				*nl += 2;
			}
			XALM_TRY(enqueue_norm_add(m, li, L, true, true, x1, m->moe_out, W, L.top, m->moe_wgt, on_tc ? m->moe_inv : nullptr, n, nl));
		}
		x = L.dwa ? m->xavg : x1;
	}
	if (want) {
		const int rows = want == 2 ? n : 1, first = want == 2 ? 0 : n - 1;
		GroupNormArgs g;
		g.y = x + (size_t) first * W; g.ldy = W;
		g.w = m->final_norm; g.groups = m->groups; g.width = W; g.eps = m->eps;
		g.x_out = m->hn;
		XALM_TRY(launch_group_norm(g, rows, s));
		(*nl)++;
		RowsEpi eh;
		eh.kind = EPI_STORE; eh.out = m->logits; eh.ldo = m->vocab;
		XALM_TRY(rows_product(m, m->hn, W, m->w_head, &m->t_head, rows, m->vocab, W, eh, nl));
	}
	return XALM_OK;
}

// ---- device layouts, cache, state, pass buffers ---------------------------------------------------------------------------------------
int finalize(SeqModel* sm) {
	Bv* m = static_cast<Bv*>(sm);
	const int W = m->width;
	const size_t C = (size_t) m->chunk;
	auto T = [&](const std::string& n) { return tensor_or_null(m, n); };
	size_t max_in = 4, max_prep = 4, max_att = 1, max_ff = 1, max_hdv = 1, max_h = 1, max_pairs = 0, max_moe_hid = 0;
	int max_tiles = 1;
	bool moe_tc = false;
	const size_t kelem = m->precision == XALM_PRECISION_F32 ? 4 : 2;
	for (size_t li = 0; li < m->layers.size(); li++) {
		Layer& L = m->layers[li];
		const std::string p = "l" + std::to_string(li) + ".";
		const int H = L.H, G = L.G, d = L.d, dv = L.dv;
		XALM_TRY(upload_vec(m, p + "norm1", &L.norm1));
		XALM_TRY(upload_vec(m, p + "dwa", &L.dwa));
		if (L.mixer == MIX_ATTENTION) {
			L.n_in = H * d + G * d + G * dv;
			XALM_TRY(upload_rows(m, {T(p + "mix.q"), T(p + "mix.k"), T(p + "mix.v")}, W, false, &L.w_in, &L.m_in));
			XALM_TRY(upload_vec(m, p + "mix.q.b", &L.bq));
			XALM_TRY(upload_vec(m, p + "mix.k.b", &L.bk));
			XALM_TRY(upload_vec(m, p + "mix.v.b", &L.bv));
			if (L.rot_dims) XALM_TRY(upload_floats(m, L.freq_host.data(), L.freq_host.size(), &L.freq));
			// the cache: pinned slots for the kept first positions, then a ring that holds one pass and the window before it
			const long long body = std::max<long long>(1, (long long) m->max_tokens - L.keep_first);
			L.ring = (int) (L.window < 0x7fffffff ? std::min<long long>(body, (long long) L.window - 1 + m->chunk) : body);
			uint8_t *kc = nullptr, *vc = nullptr;
			XALM_TRY(dev_alloc(m, &kc, (size_t) (L.keep_first + L.ring) * G * d * kelem, true));
			XALM_TRY(dev_alloc(m, &vc, (size_t) (L.keep_first + L.ring) * G * dv * kelem, true));
			L.kc = kc; L.vc = vc;
			if (!swa_pick_tq(H, G, d, dv, m->chunk) && swa_smem_bytes(H, d, dv) > 200 * 1024)
				return set_error(XALM_ERR_UNSUPPORTED, "layer %zu: attention heads need %zu bytes of shared memory", li, swa_smem_bytes(H, d, dv));
			XALM_TRY(swa_prepare(H, d, dv));
			max_hdv = std::max(max_hdv, (size_t) H * dv);
			max_h = std::max(max_h, (size_t) H);
		} else {
			L.off_k = G * d; L.off_v = 2 * G * d; L.off_g = L.off_v + H * dv; L.off_b = L.off_g + H * dv; L.off_a = L.off_b + H;
			L.n_in = L.off_a + H;
			XALM_TRY(upload_rows(m, {T(p + "mix.q"), T(p + "mix.k"), T(p + "mix.v"), T(p + "mix.g"), T(p + "mix.b"), T(p + "mix.a")}, W, false, &L.w_in, &L.m_in));
			XALM_TRY(upload_vec(m, p + "mix.q.conv", &L.cq));
			XALM_TRY(upload_vec(m, p + "mix.k.conv", &L.ck));
			XALM_TRY(upload_vec(m, p + "mix.v.conv", &L.cv));
			XALM_TRY(upload_vec(m, p + "mix.A_log", &L.A_log));
			XALM_TRY(upload_vec(m, p + "mix.dt_bias", &L.dt_bias));
			XALM_TRY(upload_vec(m, p + "mix.norm", &L.onorm));
			XALM_TRY(dev_alloc(m, &L.state, (size_t) H * d * dv, true));
			XALM_TRY(dev_alloc(m, &L.conv_state, (size_t) std::max(1, L.taps - 1) * (2 * G * d + H * dv), true));
			XALM_TRY(delta_prepare(d, dv));
			max_prep = std::max(max_prep, (size_t) 2 * G * d + H * dv + 2 * H);
		}
		XALM_TRY(upload_rows(m, {T(p + "mix.o")}, H * dv, false, &L.w_o, &L.m_o));
		max_in = std::max(max_in, (size_t) L.n_in);
		max_att = std::max(max_att, (size_t) H * dv);
		if (L.ff_kind != FF_NONE) XALM_TRY(upload_vec(m, p + "norm2", &L.norm2));
		if (L.ff_kind == FF_DENSE) {
			XALM_TRY(upload_rows(m, {T(p + "mlp.gate"), T(p + "mlp.up")}, W, true, &L.w_gu, &L.m_gu));
			XALM_TRY(upload_rows(m, {T(p + "mlp.down")}, L.ff, false, &L.w_down, &L.m_down));
			max_ff = std::max(max_ff, (size_t) L.ff);
		} else if (L.ff_kind == FF_MOE) {
			std::vector<const HostTensor*> gu, dn;
			for (int e = 0; e < L.E; e++) {
				const std::string pe = p + "mlp.e" + std::to_string(e) + ".";
				gu.push_back(T(pe + "gate"));
				gu.push_back(T(pe + "up"));
				dn.push_back(T(pe + "down"));
			}
			XALM_TRY(upload_rows(m, gu, W, true, &L.w_gu, &L.m_gu));   // all experts, one after the other
			XALM_TRY(upload_rows(m, dn, L.ff, false, &L.w_down, &L.m_down));
			XALM_TRY(upload_rows(m, {T(p + "mlp.router")}, W, false, &L.w_router, nullptr));
			XALM_TRY(moe_prepare(W, L.E, L.n_groups));
			max_pairs = std::max(max_pairs, C * L.top);
			max_moe_hid = std::max(max_moe_hid, C * L.top * L.ff);
			max_tiles = std::max(max_tiles, moe_max_tiles((int) C * L.top, L.E));
		}
	}
	XALM_TRY(group_norm_prepare(W, m->groups));
	for (Layer& L : m->layers) {
		XALM_TRY(tc_register(m, L.m_in, &L.t_in));
		XALM_TRY(tc_register(m, L.m_o, &L.t_o));
		if (L.ff_kind == FF_DENSE) {
			XALM_TRY(tc_register(m, L.m_gu, &L.t_gu));
			XALM_TRY(tc_register(m, L.m_down, &L.t_down));
		}
		// a mixture whose expert shapes the GEMM takes keeps fp16 tiles per expert for its long passes
		if (L.ff_kind == FF_MOE && m->use_tc && tune("seq_moe_tc") && tc_shape_ok(2 * L.ff, W, 2 * L.ff) && tc_shape_ok(W, L.ff, W)) {
			L.t_egu.resize((size_t) L.E);
			L.t_edown.resize((size_t) L.E);
			for (int e = 0; e < L.E; e++) {
				WMat gu = L.m_gu, dn = L.m_down; // this expert's rows of the stacked matrices
				gu.rows = 2 * L.ff;
				gu.p0 = static_cast<const uint8_t*>(L.m_gu.p0) + (size_t) e * 2 * L.ff * L.m_gu.s0;
				dn.rows = W;
				dn.p0 = static_cast<const uint8_t*>(L.m_down.p0) + (size_t) e * W * L.m_down.s0;
				XALM_TRY(tc_register(m, gu, &L.t_egu[(size_t) e]));
				XALM_TRY(tc_register(m, dn, &L.t_edown[(size_t) e]));
			}
			moe_tc = true;
		}
	}
	m->proj_ld = (int) ((max_in + 3) / 4 * 4);
	m->prep_ld = (int) ((max_prep + 3) / 4 * 4);
	m->part_cap = std::max(4 * 64, 4 * m->chunk); // one-token steps: up to 64 key splits; passes of a prompt: up to 4 per token
	XALM_TRY(dev_alloc(m, &m->hist, (m->layers.size() + 1) * C * W));
	XALM_TRY(dev_alloc(m, &m->xavg, C * W));
	XALM_TRY(dev_alloc(m, &m->proj, C * m->proj_ld));
	XALM_TRY(dev_alloc(m, &m->prep, C * m->prep_ld));
	XALM_TRY(dev_alloc(m, &m->att, C * max_att));
	XALM_TRY(dev_alloc(m, &m->y, C * W));
	XALM_TRY(dev_alloc(m, &m->ffh, C * max_ff));
	XALM_TRY(dev_alloc(m, &m->hn, C * W));
	XALM_TRY(dev_alloc(m, &m->part_o, (size_t) m->part_cap * max_hdv));
	XALM_TRY(dev_alloc(m, &m->part_ml, (size_t) m->part_cap * 2 * max_h));
	XALM_TRY(dev_alloc(m, &m->tickets, C, true));
	if (max_pairs) {
		XALM_TRY(dev_alloc(m, &m->moe_idx, max_pairs, true));
		XALM_TRY(dev_alloc(m, &m->moe_wgt, max_pairs, true));
		XALM_TRY(dev_alloc(m, &m->moe_sorted, max_pairs, true));
		XALM_TRY(dev_alloc(m, &m->moe_tiles, (size_t) 3 * max_tiles, true));
		XALM_TRY(dev_alloc(m, &m->moe_ntiles, 1, true));
		XALM_TRY(dev_alloc(m, &m->moe_hid, max_moe_hid));
		XALM_TRY(dev_alloc(m, &m->moe_out, max_pairs * W));
		if (moe_tc) {
			int max_e = 1;
			for (const Layer& L : m->layers) max_e = std::max(max_e, L.E);
			XALM_TRY(dev_alloc(m, &m->moe_off, (size_t) max_e + 1, true));
			XALM_TRY(dev_alloc(m, &m->moe_inv, max_pairs, true));
			XALM_TRY(dev_alloc(m, &m->moe_x, max_pairs * W));
			XALM_CUDA_CHECK(cudaMallocHost(&m->h_off, ((size_t) max_e + 1) * 4));
		}
	}
	return XALM_OK;
}

int release(SeqModel* sm) {
	Bv* m = static_cast<Bv*>(sm);
	for (Layer& L : m->layers)
		if (L.mixer == MIX_DELTA) {
			XALM_CUDA_CHECK(cudaMemsetAsync(L.state, 0, (size_t) L.H * L.d * L.dv * 4, m->stream));
			XALM_CUDA_CHECK(cudaMemsetAsync(L.conv_state, 0, (size_t) std::max(1, L.taps - 1) * (2 * L.G * L.d + L.H * L.dv) * 4, m->stream));
		}
	return XALM_OK;
}

// beyond the matrices: the visible K/V rows, the recurrent state read and written; of a mixture only the chosen experts are read
long long active_bytes(SeqModel* sm, long long pos) {
	Bv* m = static_cast<Bv*>(sm);
	long long b = 0;
	const long long kelem = m->precision == XALM_PRECISION_F32 ? 4 : 2, welem = m->w_bf16 ? 2 : 4;
	for (const Layer& L : m->layers) {
		if (L.mixer == MIX_ATTENTION) {
			const long long seen = L.window < 0x7fffffff ? std::min<long long>(pos + 1, (long long) L.window + L.keep_first) : pos + 1;
			b += seen * L.G * (L.d + L.dv) * kelem;
		} else b += 2ll * L.H * L.d * L.dv * 4;
		if (L.ff_kind == FF_MOE) b -= (long long) (L.E - L.top) * 3 * L.ff * m->width * welem;
	}
	return b;
}

bool state_buffer(SeqModel* sm, int layer, const float** src, size_t* count) {
	Bv* m = static_cast<Bv*>(sm);
	const Layer& L = m->layers[(size_t) layer];
	if (L.mixer != MIX_DELTA) return false;
	*src = L.state;
	*count = (size_t) L.H * L.d * L.dv;
	return true;
}

void destroy(SeqModel* sm) {
	Bv* m = static_cast<Bv*>(sm);
	for (Layer& L : m->layers)
	{
		for (TcWeight* t : {&L.t_in, &L.t_o, &L.t_gu, &L.t_down}) tc_weight_free(t);
		for (TcWeight& t : L.t_egu) tc_weight_free(&t);
		for (TcWeight& t : L.t_edown) tc_weight_free(&t);
	}
	if (m->h_off) cudaFreeHost(m->h_off);
	delete m;
}

const SeqHooks bolovik_hooks = {parse_config, finalize, enqueue_pass, release, active_bytes, state_buffer, destroy};
extern const ModelFamily bolovik_family;
int create(const char* json, int device, int max_tokens, int precision, xalm_cuda_model** out) {
	return seq_create<Bv>(&bolovik_family, &bolovik_hooks, json, device, max_tokens, precision, out);
}
const ModelFamily bolovik_family = seq_family_table("Bolovik", create);
const FamilyRegistrar bolovik_registrar(&bolovik_family);

} // namespace
} // namespace xalm
