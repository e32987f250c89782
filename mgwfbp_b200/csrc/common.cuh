// Shared device helpers: error codes, system-scope flag accesses, bounded waits, group tables.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define MGW_MAX_RANKS 16
#define MGW_MAX_CTAS 64
#define MGW_MAX_PARAM_GROUPS 16

// return codes of the host entry points
#define MGW_OK 0
#define MGW_ERR_CUDA 1
#define MGW_ERR_ARG 2
#define MGW_ERR_TOO_LARGE 3

// values of the device status word (first writer wins)
#define MGW_STATUS_OK 0
#define MGW_STATUS_TIMEOUT 1
#define MGW_STATUS_BOUNDS 2

#define MGW_CUDA_CHECK(expr)                                   \
    do {                                                       \
        cudaError_t _e = (expr);                               \
        if (_e != cudaSuccess) {                               \
            mgw_set_last_error(_e, #expr, __FILE__, __LINE__); \
            return MGW_ERR_CUDA;                               \
        }                                                      \
    } while (0)

extern "C" void mgw_set_last_error(cudaError_t e, const char* what, const char* file, int line);

// One tensor of a merged group.  `grad` is refreshed by the host whenever autograd hands out a
// new gradient tensor; `param` and `mom` never change.
struct MgwTensor {
    float* param;
    float* mom;        // null when the parameter group has no momentum
    int numel;
    int pg;            // index into the hyper-parameter table
};

// Hyper-parameters of one optimizer parameter group, read from device memory so that a learning
// rate change does not alter kernel arguments.
struct MgwHyper {
    float lr, weight_decay, momentum, dampening;
    int nesterov;
    int pad[3];
};

// A merged group in "padded vector layout": every tensor starts on a float4 boundary of the flat
// index space, voff[t] is the float4 index where tensor t starts, voff[n_tensors] == n_vec.
struct MgwGroup {
    const MgwTensor* tensors;
    float* const* grads;      // [n_tensors] current gradient pointers
    const int* voff;          // [n_tensors + 1]
    int n_tensors;
    int n_vec;
};

// mode bits of the fused kernels
#define MGW_MODE_UPDATE 1      // apply weight decay / momentum / lr to the parameters
#define MGW_MODE_WRITEBACK 2   // store the averaged gradient back into the gradient tensors
#define MGW_MODE_SUMSQ 4       // emit one partial sum of squares of the averaged gradient per CTA

#ifdef __CUDACC__

__device__ __forceinline__ uint64_t mgw_globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mgw_st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t mgw_ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// L2-coherent 16-byte accesses for memory that other GPUs read or write.
__device__ __forceinline__ float4 mgw_ld_peer(const float4* p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void mgw_st_peer(float4* p, float4 v) {
    asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
                 ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// Record the first failure in the status block (5 ints: code, peer, expected, observed, cta).
__device__ __forceinline__ void mgw_report(int* status, int code, int peer, int expected, int observed) {
    if (status == nullptr) return;
    if (atomicCAS_system(status, MGW_STATUS_OK, code) == MGW_STATUS_OK) {
        status[1] = peer;
        status[2] = expected;
        status[3] = observed;
        status[4] = blockIdx.x;
        __threadfence_system();
    }
}

// Spin until *flag >= expected or `timeout_ns` elapsed.  Returns false on timeout; never traps and
// never spins without a limit, so a missing peer leaves the context usable.
__device__ __forceinline__ bool mgw_wait_flag(const uint32_t* flag, uint32_t expected, uint64_t timeout_ns,
                                              uint32_t* observed) {
    uint32_t v = mgw_ld_acquire_sys(flag);
    if ((int32_t)(v - expected) >= 0) { *observed = v; return true; }
    const uint64_t t0 = mgw_globaltimer_ns();
    uint32_t spins = 0;
    for (;;) {
        v = mgw_ld_acquire_sys(flag);
        if ((int32_t)(v - expected) >= 0) { *observed = v; return true; }
        if ((++spins & 63u) == 0u) {
            if (mgw_globaltimer_ns() - t0 > timeout_ns) { *observed = v; return false; }
            __nanosleep(64);
        }
    }
}

// Index of the tensor that owns float4 slot v (largest t with voff[t] <= v).
__device__ __forceinline__ int mgw_find_tensor(const int* __restrict__ voff, int n_tensors, int v, int hint) {
    if (hint >= 0 && hint < n_tensors && voff[hint] <= v && v < voff[hint + 1]) return hint;
    int lo = 0, hi = n_tensors - 1;
    while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (voff[mid] <= v) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// Load the four gradient values of slot v (zero beyond the tensor's end).
__device__ __forceinline__ float4 mgw_load_grad(const MgwGroup& g, int v, int& t_hint, float scale) {
    const int t = mgw_find_tensor(g.voff, g.n_tensors, v, t_hint);
    t_hint = t;
    const int e0 = (v - g.voff[t]) << 2;
    const int n = g.tensors[t].numel;
    const float* src = g.grads[t];
    float4 r;
    if (e0 + 4 <= n) {
        r = *reinterpret_cast<const float4*>(src + e0);
    } else {
        r.x = e0 + 0 < n ? src[e0 + 0] : 0.f;
        r.y = e0 + 1 < n ? src[e0 + 1] : 0.f;
        r.z = e0 + 2 < n ? src[e0 + 2] : 0.f;
        r.w = 0.f;
    }
    r.x *= scale; r.y *= scale; r.z *= scale; r.w *= scale;
    return r;
}

__device__ __forceinline__ float mgw_sgd_scalar(float g, float& w, float* mom_slot, const MgwHyper& h, int first_step) {
    if (h.weight_decay != 0.f) g = fmaf(h.weight_decay, w, g);
    if (h.momentum != 0.f && mom_slot != nullptr) {
        float b = first_step ? g : fmaf(h.momentum, *mom_slot, (1.f - h.dampening) * g);
        *mom_slot = b;
        g = h.nesterov ? fmaf(h.momentum, b, g) : b;
    }
    w = fmaf(-h.lr, g, w);
    return w;
}

// Consume the (already averaged / scaled) gradient of slot v: optional write-back, optional SGD
// update, optional sum of squares.
__device__ __forceinline__ void mgw_consume(const MgwGroup& g, int v, float4 avg, int mode, const MgwHyper* hyper,
                                            int first_step, int& t_hint, float& sumsq) {
    const int t = mgw_find_tensor(g.voff, g.n_tensors, v, t_hint);
    t_hint = t;
    const MgwTensor te = g.tensors[t];
    const int e0 = (v - g.voff[t]) << 2;
    const int n = te.numel;
    const bool full = e0 + 4 <= n;
    if (mode & MGW_MODE_SUMSQ) {
        // padded lanes hold exact zeros, so they do not disturb the sum
        sumsq = fmaf(avg.x, avg.x, sumsq); sumsq = fmaf(avg.y, avg.y, sumsq);
        sumsq = fmaf(avg.z, avg.z, sumsq); sumsq = fmaf(avg.w, avg.w, sumsq);
    }
    if (mode & MGW_MODE_WRITEBACK) {
        float* dst = g.grads[t] + e0;
        if (full) {
            *reinterpret_cast<float4*>(dst) = avg;
        } else {
            if (e0 + 0 < n) dst[0] = avg.x;
            if (e0 + 1 < n) dst[1] = avg.y;
            if (e0 + 2 < n) dst[2] = avg.z;
        }
    }
    if (mode & MGW_MODE_UPDATE) {
        const MgwHyper h = hyper[te.pg];
        float* wp = te.param + e0;
        float* mp = te.mom ? te.mom + e0 : nullptr;
        if (full) {
            float4 w = *reinterpret_cast<float4*>(wp);
            float4 m = make_float4(0.f, 0.f, 0.f, 0.f);
            const bool use_m = (mp != nullptr) && h.momentum != 0.f;
            if (use_m && !first_step) m = *reinterpret_cast<float4*>(mp);
            mgw_sgd_scalar(avg.x, w.x, use_m ? &m.x : nullptr, h, first_step);
            mgw_sgd_scalar(avg.y, w.y, use_m ? &m.y : nullptr, h, first_step);
            mgw_sgd_scalar(avg.z, w.z, use_m ? &m.z : nullptr, h, first_step);
            mgw_sgd_scalar(avg.w, w.w, use_m ? &m.w : nullptr, h, first_step);
            *reinterpret_cast<float4*>(wp) = w;
            if (use_m) *reinterpret_cast<float4*>(mp) = m;
        } else {
            const float a[3] = {avg.x, avg.y, avg.z};
            for (int k = 0; k < 3; ++k) {
                if (e0 + k < n) {
                    float w = wp[k];
                    mgw_sgd_scalar(a[k], w, mp ? mp + k : nullptr, h, first_step);
                    wp[k] = w;
                }
            }
        }
    }
}

// Deterministic block-wide sum (fixed shuffle tree + fixed shared-memory order); result in thread 0.
__device__ __forceinline__ float mgw_block_sum(float x, float* smem /* >= 32 floats */) {
    for (int o = 16; o > 0; o >>= 1) x += __shfl_down_sync(0xffffffffu, x, o);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) smem[warp] = x;
    __syncthreads();
    float r = 0.f;
    if (threadIdx.x == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        for (int i = 0; i < nw; ++i) r += smem[i];
    }
    __syncthreads();
    return r;
}

#endif  // __CUDACC__
