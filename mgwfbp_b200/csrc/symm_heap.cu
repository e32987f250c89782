// Symmetric heap: each rank owns one device allocation of identical layout and maps every
// peer's allocation into its own address space through CUDA IPC, so kernels can load from and
// store to any GPU of the NVSwitch box with ordinary global-memory instructions.
// Handles travel between processes as opaque 64-byte blobs over the host control plane.
#include <cstdio>
#include <cstring>
#include "api.h"

static thread_local char g_last_error[512] = "";

extern "C" void mgw_set_last_error(cudaError_t e, const char* what, const char* file, int line) {
    snprintf(g_last_error, sizeof(g_last_error), "%s failed at %s:%d: %s (%s)", what, file, line,
             cudaGetErrorString(e), cudaGetErrorName(e));
    (void)cudaGetLastError();   // clear the sticky-free error so later calls start clean
}

extern "C" const char* mgw_last_error(void) { return g_last_error; }
extern "C" int mgw_version(void) { return 100; }

extern "C" int mgw_heap_create(size_t bytes, void** base_out) {
    if (base_out == nullptr || bytes == 0) return MGW_ERR_ARG;
    void* p = nullptr;
    MGW_CUDA_CHECK(cudaMalloc(&p, bytes));
    MGW_CUDA_CHECK(cudaMemset(p, 0, bytes));
    MGW_CUDA_CHECK(cudaDeviceSynchronize());
    *base_out = p;
    return MGW_OK;
}

extern "C" int mgw_heap_export(void* base, void* handle64_out) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    MGW_CUDA_CHECK(cudaIpcGetMemHandle(&h, base));
    memcpy(handle64_out, &h, sizeof(h));
    return MGW_OK;
}

extern "C" int mgw_heap_open(const void* handle64, void** peer_base_out) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    void* p = nullptr;
    MGW_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *peer_base_out = p;
    return MGW_OK;
}

extern "C" int mgw_heap_close(void* peer_base) {
    MGW_CUDA_CHECK(cudaIpcCloseMemHandle(peer_base));
    return MGW_OK;
}

extern "C" int mgw_heap_destroy(void* base) {
    MGW_CUDA_CHECK(cudaFree(base));
    return MGW_OK;
}

extern "C" int mgw_host_status_alloc(int n_ints, int** host_ptr_out) {
    int* p = nullptr;
    MGW_CUDA_CHECK(cudaHostAlloc((void**)&p, sizeof(int) * (size_t)n_ints, cudaHostAllocMapped | cudaHostAllocPortable));
    memset(p, 0, sizeof(int) * (size_t)n_ints);
    *host_ptr_out = p;
    return MGW_OK;
}

extern "C" int mgw_host_status_free(int* host_ptr) {
    MGW_CUDA_CHECK(cudaFreeHost(host_ptr));
    return MGW_OK;
}
