// Shared device helpers: error codes, system-scope flag accesses, bounded waits, group tables.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define MGW_MAX_RANKS 16
#define MGW_MAX_CTAS 296
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

// codes of the checked build's bounds word (MGW_CHECKED, see below)
#define MGW_BOUNDS_SLOT 1       // a float4 slot index outside [0, n_vec)                     {slot, n_vec}
#define MGW_BOUNDS_TENSOR 2     // the tensor found for a slot does not contain it              {slot, tensor}
#define MGW_BOUNDS_TABLE 3      // voff[] and numel of a tensor disagree                        {tensor, numel, slots}
#define MGW_BOUNDS_ELEMENT 4    // a slot starts at or beyond its tensor's last element         {slot, tensor, numel}
#define MGW_BOUNDS_STAGE 5      // a staging / inbox index beyond the region the host sized     {slot, capacity}

#ifdef __CUDACC__

// ---- checked build ----------------------------------------------------------------------------------------
// Compiled with -DMGW_CHECKED (libmgwfbp_b200_checked.so) the table-driven kernels verify every index they
// derive from a group table before using it.  A violation is recorded once per translation unit in
// g_mgw_bounds {code, a, b, c, block, thread} and the access is SKIPPED, so a wrong table costs a wrong
// result and a report, never a fault.  Without the macro the checks compile to nothing.
#ifdef MGW_CHECKED
static __device__ int g_mgw_bounds[8];
__device__ __forceinline__ bool mgw_checked(bool ok, int code, int a, int b, int c) {
    if (ok) return true;
    if (atomicCAS(&g_mgw_bounds[0], 0, code) == 0) {
        g_mgw_bounds[1] = a; g_mgw_bounds[2] = b; g_mgw_bounds[3] = c;
        g_mgw_bounds[4] = blockIdx.x; g_mgw_bounds[5] = threadIdx.x;
    }
    return false;
}
#define MGW_CHECK(cond, code, a, b, c) mgw_checked((cond), (code), (a), (b), (c))
// Host reader of this translation unit's word: out8 receives the record, which is then cleared.
#define MGW_DEFINE_BOUNDS_READER(fn)                                                        \
    extern "C" int fn(int* out8) {                                                          \
        if (out8 == nullptr) return MGW_ERR_ARG;                                            \
        MGW_CUDA_CHECK(cudaDeviceSynchronize());                                            \
        MGW_CUDA_CHECK(cudaMemcpyFromSymbol(out8, g_mgw_bounds, 8 * sizeof(int)));          \
        const int zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};                                       \
        MGW_CUDA_CHECK(cudaMemcpyToSymbol(g_mgw_bounds, zero, sizeof(zero)));               \
        return MGW_OK;                                                                      \
    }
#else
#define MGW_CHECK(cond, code, a, b, c) (true)
#define MGW_DEFINE_BOUNDS_READER(fn)                                  \
    extern "C" int fn(int* out8) {                                    \
        if (out8 == nullptr) return MGW_ERR_ARG;                      \
        for (int i = 0; i < 8; ++i) out8[i] = 0;                      \
        return MGW_OK;                                                \
    }
#endif

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
    if (!MGW_CHECK(v >= 0 && v < g.n_vec, MGW_BOUNDS_SLOT, v, g.n_vec, 0)) return make_float4(0.f, 0.f, 0.f, 0.f);
    const int t = mgw_find_tensor(g.voff, g.n_tensors, v, t_hint);
    t_hint = t;
    if (!MGW_CHECK(g.voff[t] <= v && v < g.voff[t + 1], MGW_BOUNDS_TENSOR, v, t, 0)) return make_float4(0.f, 0.f, 0.f, 0.f);
    const int e0 = (v - g.voff[t]) << 2;
    const int n = g.tensors[t].numel;
    if (!MGW_CHECK(e0 < n, MGW_BOUNDS_ELEMENT, v, t, n)) return make_float4(0.f, 0.f, 0.f, 0.f);
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
    if (!MGW_CHECK(v >= 0 && v < g.n_vec, MGW_BOUNDS_SLOT, v, g.n_vec, 0)) return;
    const int t = mgw_find_tensor(g.voff, g.n_tensors, v, t_hint);
    t_hint = t;
    if (!MGW_CHECK(g.voff[t] <= v && v < g.voff[t + 1], MGW_BOUNDS_TENSOR, v, t, 0)) return;
    const MgwTensor te = g.tensors[t];
    const int e0 = (v - g.voff[t]) << 2;
    const int n = te.numel;
    if (!MGW_CHECK(e0 < n, MGW_BOUNDS_ELEMENT, v, t, n)) return;
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

// ---- batched streaming access -------------------------------------------------------------------------
// A thread walks slots v0, v0 + stride, ..., v0 + (U-1) * stride per iteration.  MgwCursor caches the
// tensor that owns them; while all U slots are whole float4s of that one tensor (the common case
// for convolution and linear weights) the loads of a batch are issued back to back with no table
// lookups in between, so U independent 16-byte requests per operand are in flight per thread.

struct MgwCursor {
    int t;         // cached tensor index (-1: nothing cached yet)
    int vbeg;      // its first slot
    int vfull;     // first slot not entirely inside the tensor: vbeg + numel / 4
    int vend;      // first slot of the next tensor
    int numel, pg;
    float* grad;
    float* param;
    float* mom;
};

__device__ __forceinline__ MgwCursor mgw_cursor() {
    MgwCursor c;
    c.t = -1; c.vbeg = 0; c.vfull = 0; c.vend = 0; c.numel = 0; c.pg = 0;
    c.grad = nullptr; c.param = nullptr; c.mom = nullptr;
    return c;
}

__device__ __forceinline__ void mgw_seek(const MgwGroup& g, int v, MgwCursor& c) {
    const int t = mgw_find_tensor(g.voff, g.n_tensors, v, c.t + 1);      // walking forward: the next tensor is the likely one
    const MgwTensor te = g.tensors[t];
    c.t = t;
    c.vbeg = g.voff[t];
    c.vend = g.voff[t + 1];
    c.numel = te.numel;
    c.vfull = c.vbeg + (te.numel >> 2);
    c.pg = te.pg;
    c.grad = g.grads[t];
    c.param = te.param;
    c.mom = te.mom;
    if (!MGW_CHECK(c.vbeg <= v && v < c.vend && c.vbeg + ((te.numel + 3) >> 2) == c.vend, MGW_BOUNDS_TABLE, t, te.numel,
                   c.vend - c.vbeg))
        c.vfull = c.vbeg;            // no slot qualifies for the table-free path; the per-slot path re-checks each one
}

// True when slots v0 .. v0 + (U-1) * stride are all below `vlimit` and whole float4s of one tensor; positions the cursor.
template <int U>
__device__ __forceinline__ bool mgw_batch_is_plain(const MgwGroup& g, int v0, int stride, int vlimit, MgwCursor& c) {
    const int vl = v0 + (U - 1) * stride;
    if (vl >= vlimit) return false;
    if (v0 < c.vbeg || v0 >= c.vend) mgw_seek(g, v0, c);
    return vl < c.vfull;
}

template <int U>
__device__ __forceinline__ void mgw_load_grad_batch(const MgwGroup& g, int v0, int stride, int vlimit, MgwCursor& c,
                                                    float scale, float4 (&x)[U]) {
    if (mgw_batch_is_plain<U>(g, v0, stride, vlimit, c)) {
        const float4* src = reinterpret_cast<const float4*>(c.grad) + (v0 - c.vbeg);
#pragma unroll
        for (int k = 0; k < U; ++k) x[k] = src[k * stride];
#pragma unroll
        for (int k = 0; k < U; ++k) { x[k].x *= scale; x[k].y *= scale; x[k].z *= scale; x[k].w *= scale; }
    } else {
        int hint = c.t;
#pragma unroll
        for (int k = 0; k < U; ++k)
            if (v0 + k * stride < vlimit) x[k] = mgw_load_grad(g, v0 + k * stride, hint, scale);
    }
}

template <int U>
__device__ __forceinline__ void mgw_consume_batch(const MgwGroup& g, int v0, int stride, int vlimit, MgwCursor& c,
                                                  const float4 (&x)[U], int mode, const MgwHyper* hyper, int first_step,
                                                  float& sumsq) {
    if (!mgw_batch_is_plain<U>(g, v0, stride, vlimit, c)) {
        int hint = c.t;
#pragma unroll
        for (int k = 0; k < U; ++k)
            if (v0 + k * stride < vlimit) mgw_consume(g, v0 + k * stride, x[k], mode, hyper, first_step, hint, sumsq);
        return;
    }
    const int off = v0 - c.vbeg;
    if (mode & MGW_MODE_SUMSQ) {
#pragma unroll
        for (int k = 0; k < U; ++k) {
            sumsq = fmaf(x[k].x, x[k].x, sumsq); sumsq = fmaf(x[k].y, x[k].y, sumsq);
            sumsq = fmaf(x[k].z, x[k].z, sumsq); sumsq = fmaf(x[k].w, x[k].w, sumsq);
        }
    }
    if (mode & MGW_MODE_WRITEBACK) {
        float4* dst = reinterpret_cast<float4*>(c.grad) + off;
#pragma unroll
        for (int k = 0; k < U; ++k) dst[k * stride] = x[k];
    }
    if (mode & MGW_MODE_UPDATE) {
        const MgwHyper h = hyper[c.pg];
        float4* wp = reinterpret_cast<float4*>(c.param) + off;
        float4* mp = reinterpret_cast<float4*>(c.mom) + off;
        const bool use_m = (c.mom != nullptr) && h.momentum != 0.f;
        float4 w[U], m[U];
#pragma unroll
        for (int k = 0; k < U; ++k) w[k] = wp[k * stride];
#pragma unroll
        for (int k = 0; k < U; ++k) m[k] = (use_m && !first_step) ? mp[k * stride] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < U; ++k) {
            mgw_sgd_scalar(x[k].x, w[k].x, use_m ? &m[k].x : nullptr, h, first_step);
            mgw_sgd_scalar(x[k].y, w[k].y, use_m ? &m[k].y : nullptr, h, first_step);
            mgw_sgd_scalar(x[k].z, w[k].z, use_m ? &m[k].z : nullptr, h, first_step);
            mgw_sgd_scalar(x[k].w, w[k].w, use_m ? &m[k].w : nullptr, h, first_step);
        }
#pragma unroll
        for (int k = 0; k < U; ++k) wp[k * stride] = w[k];
        if (use_m) {
#pragma unroll
            for (int k = 0; k < U; ++k) mp[k * stride] = m[k];
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
