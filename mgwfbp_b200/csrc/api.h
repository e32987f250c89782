// C ABI of libmgwfbp_b200.so.  Every entry point returns MGW_OK (0) or an MGW_ERR_* code;
// mgw_last_error() gives the text of the most recent failure on the calling thread.
// The header is C++ (common.cuh needs cuda_runtime.h); the symbols have C linkage and can be bound from any language
// through the shared library (the package itself uses ctypes).
#pragma once
#include <stddef.h>
#include <stdint.h>
#include "common.cuh"

#ifdef __cplusplus
extern "C" {
#endif

const char* mgw_last_error(void);
int mgw_version(void);

void mgw_set_last_error_text(const char* text);

// ---- symmetric heap (symm_heap.cu): one region per rank, mapped into every peer ---------------------
// VMM flavour: cuMemCreate memory shared as POSIX file descriptors, optionally bound to an NVSwitch multicast object.
int mgw_vmm_supported(int* out2);                                    // {vmm + fd handles, multicast}
int mgw_vmm_create(size_t bytes, int world, int want_multicast, void** heap_out, void** base_out, size_t* bytes_out);
int mgw_vmm_export_fd(void* heap, int* fd_out);
int mgw_vmm_import_peer(void* heap, int peer, int fd, void** peer_base_out);
int mgw_vmm_mc_create(void* heap, int world, int* fd_out);
int mgw_vmm_mc_import(void* heap, int fd);
int mgw_vmm_mc_add_device(void* heap);
int mgw_vmm_mc_bind(void* heap, void** mc_base_out);
int mgw_vmm_destroy(void* heap, int what);                           // what: 0 everything, 1 the multicast part only
// IPC flavour: cudaMalloc + cudaIpc handles.
int mgw_heap_create(size_t bytes, void** base_out);
int mgw_heap_export(void* base, void* handle64_out);                 // 64-byte IPC handle
int mgw_heap_open(const void* handle64, void** peer_base_out);      // enables peer access lazily
int mgw_heap_close(void* peer_base);
int mgw_heap_destroy(void* base);
int mgw_host_status_alloc(int n_ints, int** host_ptr_out);           // pinned, device-visible status block
int mgw_host_status_free(int* host_ptr);

// ---- fused all-reduce (+ SGD update) of one merged group (allreduce_fused.cu) ---------------------
#define MGW_ALGO_ONESHOT 0
#define MGW_ALGO_TWOSHOT 1
#define MGW_ALGO_NVLS 2

typedef struct {
    MgwGroup group;
    float* stage[MGW_MAX_RANKS];        // every rank's staging area of this group (own rank included)
    uint32_t* flags[MGW_MAX_RANKS];     // every rank's flag block
    uint32_t* epoch;                    // this rank's per-CTA launch counters [MGW_MAX_CTAS]
    float* mc_stage;                    // NVSwitch multicast address of the staging area, or null
    const MgwHyper* hyper;
    float* sumsq_partials;              // [n_ctas] or null
    int* status;                        // 8 ints, host-visible
    int rank, world;
    int algo, n_ctas, n_threads;
    int mode, first_step;
    int inbox_stride;                   // one-shot: float4 slots between consecutive inbox rows (>= n_vec)
    int stage_slots;                    // two-shot / NVLS: float4 slots the staging area holds (>= n_vec)
    int max_pieces;                     // two-shot / NVLS: the chunk of a CTA is processed in at most this many pieces ...
    int piece_slots;                    // ... of at least this many float4 slots (1, anything: no pipelining)
    float grad_scale;                   // multiplies the summed gradient together with 1/world (1 / loss scale)
    int skip_pack;                      // two-shot / NVLS: the staging area was already filled (device-to-device copies)
    unsigned long long timeout_ns;
} MgwAllreduceArgs;

int mgw_allreduce_group(const MgwAllreduceArgs* args, void* stream);
// Checked build only (-DMGW_CHECKED): first index violation recorded by the kernels of allreduce_fused.cu /
// multi_tensor_sgd.cu as {code, a, b, c, block, thread, 0, 0} (MGW_BOUNDS_*), cleared by the call.  All zeros otherwise.
int mgw_bounds_allreduce(int* out8);
int mgw_bounds_sgd(int* out8);
// Checked build only: per-CTA phase stamps (ns since CTA start) of the most recent two-shot / NVLS launch.
int mgw_phase_times(unsigned long long* out, int n_ctas);
size_t mgw_flag_block_bytes(void);
// staging bytes one rank needs for a group of n_vec float4 slots under `algo`
size_t mgw_stage_bytes(int algo, int n_vec, int world);

// ---- standalone multi-tensor SGD (multi_tensor_sgd.cu) ----------------------------------------------
// grad_scale multiplies every gradient first; clip_coef (device pointer, may be null) multiplies it too.
int mgw_multi_tensor_sgd(const MgwGroup* group, const MgwHyper* hyper, const float* clip_coef, float grad_scale,
                         int first_step, int mode, float* sumsq_partials, int n_ctas, void* stream);
// Sum `n` partial sums of squares in a fixed order; writes total norm to out[0] and
// min(1, max_norm / (norm + 1e-6)) to out[1].
int mgw_clip_coef(const float* partials, int n, float max_norm, float* out2, void* stream);
// Sum of squares of the gradients of a group (one partial per CTA, deterministic).
int mgw_group_sumsq(const MgwGroup* group, float* partials, int n_ctas, void* stream);

// ---- stem convolution input rearrangement (stem_s2d.cu) ---------------------------------------------
// x [N, H, W, 3] channels-last image batch (H, W even) -> out [N, H/2 + 3, W/2 + 3, 12], zero padded:
// out[n, j, i, p*6 + q*3 + c] = x[n, 2j + p - 4, 2i + q - 4, c].
int mgw_s2d_stem_input(const float* x, float* out, int N, int H, int W, void* stream);

#ifdef __cplusplus
}
#endif
