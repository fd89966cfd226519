// abi.cu — the part of the C ABI (include/xalm_cuda.h) that belongs to no model family: diagnostics, pinned host memory, the
// tuning knobs, the family registry (family.h) and the handle-based entry points, each forwarded through the family table the
// handle names.  The families' own translation units (xalm_cuda.cu: Llama/Mistral; nabalix.cu) never export those symbols.
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <string>
#include <vector>

#include "family.h"
#include "host/json.h"

namespace xalm {

thread_local std::string g_last_error;

int set_error(int status, const char* fmt, ...) {
	char buf[1024];
	va_list ap;
	va_start(ap, fmt);
	vsnprintf(buf, sizeof buf, fmt, ap);
	va_end(ap);
	g_last_error = buf;
	return status;
}

// ---------------------------------------------------------------------------------------------------------
// tuning knobs (xalm_cuda_tune): integers looked up by name, so GPU sweeps need no recompilation
// ---------------------------------------------------------------------------------------------------------
static std::map<std::string, int>& tuning() {
	static std::map<std::string, int> t = {
	    {"pdl", 1},          // programmatic dependent launch between the kernels of a token
	    {"graph", 1},        // replay a captured CUDA graph per token
	    {"attn_splits", 0},  // 0 = auto (~1 CTA per SM, at most 32 splits per kv head)
	    {"attn_min_split", 128},
	    {"mv_cfg_rows", 0},  // 0 = auto, 1 = force config A (R4 KS1 NW4), 2 = force config B (R2 KS4 NW8)
	    {"mega", 0},         // EXPERIMENTAL, measured slower than the kernel-per-op path (profiles/r2_token_kernel.md): one persistent kernel per
	                         // token (decode_mega.cu) when the model allows — single GPU, integer weight formats
	    {"mega_smem_kb", 170}, // shared memory per CTA the token kernel may take: the ring gets what the staged activations leave (3 stages on a
	                           // 7B model: deeper rings measured no faster), the rest of the 228 KB stays L1
	    {"mega_ns_max", 16},
	    {"mega_quiet", 1},   // the token kernel's producer pauses while the consumers hand over between phases
	    {"mega_coop", 1},    // cooperative launch of the token kernel
	    {"mega_timeline", 0}, // record per-phase %globaltimer stamps (xalm_cuda_mega_timeline)
	    {"tma", 1},          // stream weights with cp.async.bulk into a shared-memory ring (matvec_tma.cuh)
	    {"idp", 1},          // integer weight formats: integer-dot consumers (matvec_idp.cuh) instead of the float ones
	    {"tma_smem_kb", 100}, // shared-memory budget per CTA for the TMA kernel (two kernels co-reside under PDL)
	    {"tma_rc_small", 8}, // rows per tile when the matrix has few rows (Wo, W2)
	    {"tma_xstage_max_kb", 32}, // rows longer than this (in fp32 bytes) are not staged in smem when there is no norm
	    {"tma_norm_kw4", 0}, {"tma_norm_smem_kb", 72},
	    {"tma_rc", 0},       // 0 = auto, else force rows per tile (4 or 8)
	    {"tma_ns_max", 4},   // most ring stages
	    {"tma_ctas_per_sm", 2},
	    {"tma_short_rows", 1}, // rows of <= 64 pieces without a norm prologue: 16-row tiles with 1-2 K-slices (all lanes busy)
	    {"tma_grid_even", 0}, // percent: shrink the persistent grid down to this fraction of the full one if that makes tiles % grid == 0
	    {"tp_fused", 1},     // tensor parallel: fuse the two per-layer exchanges into the matvec kernels (push over NVLink + receive in the next prologue)
	    {"idp_per_sm", 2},
	    {"mma", 2},         // integer formats on the tensor-core matvec (fragment tiles + mma.sync int8, matvec_mma.cuh): 0 = never (unit layout + dp4a), 1 = all six, 2 = the 4/5-bit formats, and the 8-bit ones under tensor parallelism (measured on one GPU: q4_0 1.68 vs 1.86 ms/token; q8_0 1.90 vs 1.86)
    {"idp_ng", 0},      // consumer groups per CTA of the integer-dot matvec: 0 = by format, 2 = one 17-warp CTA per SM, 1 = two 9-warp CTAs
	    {"tail_prefetch_mb", 8}, // each decode kernel pulls this many MB of the NEXT kernel's first weights into L2 once its own loads are issued
	    {"prefill_split", 3}, // batched prefill operand precision: 1 = fp16 x fp16 (fastest; logits drift ~4e-2 over 32 layers), 2 = hi+lo fp16
	                          // activations, 3 = hi+lo on activations, weights and attention operands (default: logits within ~1e-3 of the decode path)
	    {"seq_graph", 1},     // config.json families: replay a captured CUDA graph for one-token steps
	    {"seq_chunk", 256},   // config.json families: most positions one pass of a prompt covers (longer steps are cut)
	    {"seq_tc", 1},        // config.json families, 16-bit serving mode: passes of many tokens run their matrix products on the tcgen05 GEMM where the
	                          // shapes allow; 1 = activations as one fp16 plane, 2 = hi + lo planes (fp32-grade), 0 = fp32 FMA kernels only
	    {"seq_tc_min", 32},   // fewest tokens in a pass for that path
	    {"seq_moe_tc", 1},    // config.json families with expert mixtures, 16-bit serving mode: long passes gather each expert's rows and run them on the
	                          // tcgen05 GEMM (one small device-to-host copy of the experts' row counts per mixture layer and pass); 0 = fp32 FMA tiles
	    {"seq_overlap", 1},   // config.json families: mixers of a layer that do not depend on one another run on two streams (two branches of the graph)
	};
	return t;
}
int tune(const char* k) {
	const char* e = nullptr;
	std::string env = std::string("XALM_") + k;
	for (auto& ch : env) ch = (char) toupper(ch);
	if ((e = getenv(env.c_str()))) return atoi(e);
	return tuning()[k];
}


// ---------------------------------------------------------------------------------------------------------
// family registry
// ---------------------------------------------------------------------------------------------------------
static std::vector<const ModelFamily*>& families() {
	static std::vector<const ModelFamily*> f;
	return f;
}
void register_family(const ModelFamily* f) { families().push_back(f); }
const ModelFamily* find_family(const char* name) {
	for (const ModelFamily* f : families())
		if (!strcmp(f->name, name)) return f;
	return nullptr;
}

static const ModelFamily* family_of(const xalm_cuda_model* m) { return m ? reinterpret_cast<const ModelHead*>(m)->family : nullptr; }

} // namespace xalm

using namespace xalm;

// forward a handle-based call through the family table
#define XALM_DISPATCH(member, ...)                                                                                  \
	do {                                                                                                            \
		const ModelFamily* f_ = family_of(m);                                                                       \
		if (!f_) return set_error(XALM_ERR_INVALID, "model is NULL");                                               \
		if (!f_->member) return set_error(XALM_ERR_UNSUPPORTED, "the %s family has no " #member, f_->name);          \
		return f_->member(__VA_ARGS__);                                                                             \
	} while (0)

extern "C" {

int xalm_cuda_abi_version(void) { return XALM_CUDA_ABI_VERSION; }
const char* xalm_cuda_last_error(void) { return g_last_error.c_str(); }

int xalm_cuda_device_count(int* count) {
	if (!count) return set_error(XALM_ERR_INVALID, "count is NULL");
	cudaError_t e = cudaGetDeviceCount(count);
	if (e != cudaSuccess) return set_error(XALM_ERR_CUDA, "cudaGetDeviceCount failed: %s", cudaGetErrorString(e));
	return XALM_OK;
}

int xalm_cuda_tune(const char* key, int value) {
	if (!key || !tuning().count(key)) return set_error(XALM_ERR_INVALID, "unknown tuning key '%s'", key ? key : "(null)");
	tuning()[key] = value;
	return XALM_OK;
}

void* xalm_cuda_host_alloc(size_t nbytes) {
	void* p = nullptr;
	cudaError_t e = cudaMallocHost(&p, nbytes ? nbytes : 16);
	if (e != cudaSuccess) { set_error(XALM_ERR_CUDA, "cudaMallocHost(%zu) failed: %s", nbytes, cudaGetErrorString(e)); return nullptr; }
	return p;
}
void xalm_cuda_host_free(void* p) {
	if (p) cudaFreeHost(p);
}

int xalm_cuda_family_count(void) { return (int) families().size(); }
const char* xalm_cuda_family_name(int index) {
	return index >= 0 && index < (int) families().size() ? families()[(size_t) index]->name : nullptr;
}

int xalm_cuda_create(const xalm_config* cfg, int device, int tp_rank, int tp_size, xalm_cuda_model** out) {
	const ModelFamily* f = find_family("Llama");
	if (!f || !f->create_pod) return set_error(XALM_ERR_UNSUPPORTED, "this build carries no family that is created from an xalm_config");
	return f->create_pod(cfg, device, tp_rank, tp_size, out);
}

int xalm_cuda_create_json(const char* config_json, int device, int max_tokens, int precision, xalm_cuda_model** out) {
	if (!config_json || !out) return set_error(XALM_ERR_INVALID, "config_json/out is NULL");
	*out = nullptr;
	std::string arch;
	try {
		const xjson::Value v = xjson::Parser::parse(config_json, strlen(config_json));
		const xjson::Value* a = v.find("architecture");
		if (!a || a->kind != xjson::Value::String) return set_error(XALM_ERR_INVALID, "config.json names no architecture");
		arch = a->str;
	} catch (const std::exception& e) {
		return set_error(XALM_ERR_INVALID, "config.json: %s", e.what());
	}
	const ModelFamily* f = find_family(arch.c_str());
	if (!f || !f->create_json) return set_error(XALM_ERR_UNSUPPORTED, "unsupported model architecture: %s", arch.c_str());
	if (precision != XALM_PRECISION_BF16 && precision != XALM_PRECISION_F32) return set_error(XALM_ERR_INVALID, "precision %d", precision);
	return f->create_json(config_json, device, max_tokens, precision, out);
}

int xalm_cuda_upload_tensor(xalm_cuda_model* m, const char* name, int type_id, const int* shape, int rank, const void* data, size_t nbytes) {
	XALM_DISPATCH(upload_tensor, m, name, type_id, shape, rank, data, nbytes);
}
int xalm_cuda_shard_range(xalm_cuda_model* m, const char* name, int* range4) { XALM_DISPATCH(shard_range, m, name, range4); }
int xalm_cuda_upload_tensor_shard(xalm_cuda_model* m, const char* name, int type_id, const int* shape, int rank, const int* range4,
                                  const void* data, size_t nbytes) {
	XALM_DISPATCH(upload_tensor_shard, m, name, type_id, shape, rank, range4, data, nbytes);
}
int xalm_cuda_finalize(xalm_cuda_model* m) { XALM_DISPATCH(finalize, m); }
void xalm_cuda_destroy(xalm_cuda_model* m) {
	const ModelFamily* f = family_of(m);
	if (f && f->destroy) f->destroy(m);
}
int xalm_cuda_comm_init(xalm_cuda_model* m, const void* id128) { XALM_DISPATCH(comm_init, m, id128); }
int xalm_cuda_ipc_export(xalm_cuda_model* m, void* handle64) { XALM_DISPATCH(ipc_export, m, handle64); }
int xalm_cuda_ipc_import(xalm_cuda_model* m, const void* handles) { XALM_DISPATCH(ipc_import, m, handles); }
int xalm_cuda_set_stream(xalm_cuda_model* m, void* cuda_stream) { XALM_DISPATCH(set_stream, m, cuda_stream); }
int xalm_cuda_forward(xalm_cuda_model* m, int token, int pos, int mode, float* logits_host) {
	XALM_DISPATCH(forward, m, token, pos, mode, logits_host);
}
int xalm_cuda_forward_argmax(xalm_cuda_model* m, int token, int pos, int* next_token) { XALM_DISPATCH(forward_argmax, m, token, pos, next_token); }
int xalm_cuda_forward_async(xalm_cuda_model* m, int token, int pos, int mode) { XALM_DISPATCH(forward_async, m, token, pos, mode); }
int xalm_cuda_sync(xalm_cuda_model* m) { XALM_DISPATCH(sync, m); }
int xalm_cuda_prefill(xalm_cuda_model* m, const int* tokens, int n, int pos0, int want_logits, float* logits_host, const int* targets,
                      float* probs_host) {
	XALM_DISPATCH(prefill, m, tokens, n, pos0, want_logits, logits_host, targets, probs_host);
}
int xalm_cuda_prefill_async(xalm_cuda_model* m, const int* tokens, int n, int pos0, int want_logits) {
	XALM_DISPATCH(prefill_async, m, tokens, n, pos0, want_logits);
}
float* xalm_cuda_logits_host(xalm_cuda_model* m) {
	const ModelFamily* f = family_of(m);
	return f && f->logits_host ? f->logits_host(m) : nullptr;
}
int xalm_cuda_active_bytes(xalm_cuda_model* m, long long pos, long long* bytes) { XALM_DISPATCH(active_bytes, m, pos, bytes); }
int xalm_cuda_last_launch_count(xalm_cuda_model* m, int* n) { XALM_DISPATCH(last_launch_count, m, n); }
int xalm_cuda_read_state(xalm_cuda_model* m, int which, float* dst, size_t n) { XALM_DISPATCH(read_state, m, which, dst, n); }
int xalm_cuda_read_kv(xalm_cuda_model* m, int layer, int which, uint16_t* dst, size_t n_elems) {
	XALM_DISPATCH(read_kv, m, layer, which, dst, n_elems);
}
int xalm_cuda_mega_timeline(xalm_cuda_model* m, unsigned long long* out, size_t cap_words, int* n_phases, int* grid) {
	XALM_DISPATCH(mega_timeline, m, out, cap_words, n_phases, grid);
}
int xalm_cuda_release(xalm_cuda_model* m) { XALM_DISPATCH(release, m); }
int xalm_cuda_expected_tensor(xalm_cuda_model* m, int index, char* name, size_t name_cap, int* shape4, int* rank) {
	XALM_DISPATCH(expected_tensor, m, index, name, name_cap, shape4, rank);
}
int xalm_cuda_model_info(xalm_cuda_model* m, const char* key, long long* value) { XALM_DISPATCH(info, m, key, value); }

} // extern "C"
