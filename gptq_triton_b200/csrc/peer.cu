// Exchange buffers for the tensor-parallel epilogue: plain cudaMalloc allocations (outside any
// caching allocator, so that a CUDA IPC handle names exactly this buffer), exported to and opened
// by the other ranks of the node.  Opening enables peer access lazily.
#include <cuda_runtime.h>

#include <cstring>

#include "../../include/gptq_b200.h"
#include "common.cuh"

using namespace gptq;

extern "C" {

int gptq_peer_alloc(size_t bytes, void **ptr) {
	if (!ptr || bytes == 0) return GPTQ_ERR_INVALID;
	void *p = nullptr;
	cudaError_t e = cudaMalloc(&p, bytes);
	if (e != cudaSuccess) return cuda_status(e);
	e = cudaMemset(p, 0, bytes);
	if (e != cudaSuccess) {
		cudaFree(p);
		return cuda_status(e);
	}
	*ptr = p;
	return GPTQ_OK;
}

int gptq_peer_free(void *ptr) { return ptr ? cuda_status(cudaFree(ptr)) : GPTQ_OK; }

int gptq_peer_export(void *ptr, void *handle64) {
	if (!ptr || !handle64) return GPTQ_ERR_INVALID;
	static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
	cudaIpcMemHandle_t h;
	cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
	if (e != cudaSuccess) return cuda_status(e);
	std::memcpy(handle64, &h, 64);
	return GPTQ_OK;
}

int gptq_peer_open(const void *handle64, void **ptr) {
	if (!handle64 || !ptr) return GPTQ_ERR_INVALID;
	cudaIpcMemHandle_t h;
	std::memcpy(&h, handle64, 64);
	void *p = nullptr;
	cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
	if (e != cudaSuccess) return cuda_status(e);
	*ptr = p;
	return GPTQ_OK;
}

int gptq_peer_close(void *ptr) { return ptr ? cuda_status(cudaIpcCloseMemHandle(ptr)) : GPTQ_OK; }

}   // extern "C"
