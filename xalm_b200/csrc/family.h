// family.h — the model registry behind the opaque handle of include/xalm_cuda.h.
//
// A model family (Llama/Mistral-style transformers, Nabalix, ...) is a table of the handle-based entry points.  Every handle
// starts with a ModelHead naming its family; abi.cu exports the C symbols once and forwards each call through that table, so
// a host program drives every family with the same calls (upload_tensor -> finalize -> forward / prefill -> release -> destroy)
// and a family lives in translation units of its own: the library can be linked with any subset of them.
//
// Families described by a config.json ("architecture": "<name>") register a create_json function under that name
// (xalm_cuda_create_json looks it up); the Llama family keeps its POD constructor xalm_cuda_create (Config, model.h:25-42).
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "../../include/xalm_cuda.h"

namespace xalm {

struct ModelFamily {
	const char* name;
	// NULL members answer XALM_ERR_UNSUPPORTED ("<family> has no <call>")
	int (*create_json)(const char* config_json, int device, int max_tokens, int precision, xalm_cuda_model** out);
	int (*upload_tensor)(xalm_cuda_model*, const char* name, int type_id, const int* shape, int rank, const void* data, size_t nbytes);
	int (*shard_range)(xalm_cuda_model*, const char* name, int* range4);
	int (*upload_tensor_shard)(xalm_cuda_model*, const char* name, int type_id, const int* shape, int rank, const int* range4, const void* data,
	                           size_t nbytes);
	int (*finalize)(xalm_cuda_model*);
	void (*destroy)(xalm_cuda_model*);
	int (*comm_init)(xalm_cuda_model*, const void* id128);
	int (*ipc_export)(xalm_cuda_model*, void* handle64);
	int (*ipc_import)(xalm_cuda_model*, const void* handles);
	int (*set_stream)(xalm_cuda_model*, void* cuda_stream);
	int (*forward)(xalm_cuda_model*, int token, int pos, int mode, float* logits_host);
	int (*forward_argmax)(xalm_cuda_model*, int token, int pos, int* next_token);
	int (*forward_async)(xalm_cuda_model*, int token, int pos, int mode);
	int (*sync)(xalm_cuda_model*);
	int (*prefill)(xalm_cuda_model*, const int* tokens, int n, int pos0, int want_logits, float* logits_host, const int* targets, float* probs_host);
	int (*prefill_async)(xalm_cuda_model*, const int* tokens, int n, int pos0, int want_logits);
	float* (*logits_host)(xalm_cuda_model*);
	int (*active_bytes)(xalm_cuda_model*, long long pos, long long* bytes);
	int (*last_launch_count)(xalm_cuda_model*, int* n);
	int (*read_state)(xalm_cuda_model*, int which, float* dst, size_t n);
	int (*read_kv)(xalm_cuda_model*, int layer, int which, uint16_t* dst, size_t n_elems);
	int (*mega_timeline)(xalm_cuda_model*, unsigned long long* out, size_t cap_words, int* n_phases, int* grid);
	// sequence state: give back what the running sequence holds in the cache / recurrent state; the next call starts at position 0
	int (*release)(xalm_cuda_model*);
	// the tensors the family expects, for loaders: index -> name and element shape; XALM_ERR_INVALID past the last one
	int (*expected_tensor)(xalm_cuda_model*, int index, char* name, size_t name_cap, int* shape4, int* rank);
	// integer properties by name ("vocab_size", "n_layers", ...)
	int (*info)(xalm_cuda_model*, const char* key, long long* value);
	// families built from the POD xalm_config (xalm_cuda_create): the Llama family only
	int (*create_pod)(const xalm_config* cfg, int device, int tp_rank, int tp_size, xalm_cuda_model** out);
};

struct ModelHead {
	const ModelFamily* family;
};

// called from a static initialiser of the family's translation unit
void register_family(const ModelFamily* f);
const ModelFamily* find_family(const char* name);

struct FamilyRegistrar {
	explicit FamilyRegistrar(const ModelFamily* f) { register_family(f); }
};

// integer tuning knobs (xalm_cuda_tune); an XALM_<KEY> environment variable overrides the stored value
int tune(const char* key);

} // namespace xalm
