// llama_names.h — included first by xalm_cuda.cu.  The handle-based entry points of include/xalm_cuda.h are exported once, by
// abi.cu, which forwards each call through the family table of the handle (family.h).  This translation unit holds the
// Llama/Mistral family's implementations of them, under these names; they enter the family table at the end of the file.
#pragma once
#define xalm_cuda_create xalm_llama_create
#define xalm_cuda_upload_tensor xalm_llama_upload_tensor
#define xalm_cuda_shard_range xalm_llama_shard_range
#define xalm_cuda_upload_tensor_shard xalm_llama_upload_tensor_shard
#define xalm_cuda_finalize xalm_llama_finalize
#define xalm_cuda_destroy xalm_llama_destroy
#define xalm_cuda_comm_init xalm_llama_comm_init
#define xalm_cuda_ipc_export xalm_llama_ipc_export
#define xalm_cuda_ipc_import xalm_llama_ipc_import
#define xalm_cuda_set_stream xalm_llama_set_stream
#define xalm_cuda_forward xalm_llama_forward
#define xalm_cuda_forward_argmax xalm_llama_forward_argmax
#define xalm_cuda_forward_async xalm_llama_forward_async
#define xalm_cuda_sync xalm_llama_sync
#define xalm_cuda_prefill xalm_llama_prefill
#define xalm_cuda_prefill_async xalm_llama_prefill_async
#define xalm_cuda_logits_host xalm_llama_logits_host
#define xalm_cuda_active_bytes xalm_llama_active_bytes
#define xalm_cuda_last_launch_count xalm_llama_last_launch_count
#define xalm_cuda_read_state xalm_llama_read_state
#define xalm_cuda_read_kv xalm_llama_read_kv
#define xalm_cuda_mega_timeline xalm_llama_mega_timeline
