// Multi-tensor momentum SGD: one launch updates every parameter of a model (or of one merged
// group).  Replaces the per-tensor elementwise launches of torch.optim.SGD.step on the 1-GPU
// path, after gradient accumulation, and after a global-norm clip (the clip coefficient is read
// from device memory, so no host round trip separates the norm from the update).
#include <atomic>
#include "api.h"

template <int U, int MIN_BLOCKS>                          // U: float4 slots per operand a thread keeps in flight
__global__ void __launch_bounds__(512, MIN_BLOCKS)
mgw_multi_tensor_sgd_kernel(MgwGroup g, const MgwHyper* __restrict__ hyper, const float* __restrict__ clip_coef,
                            float grad_scale, int first_step, int mode, float* __restrict__ sumsq_partials) {
    __shared__ float red[32];
    float scale = grad_scale;
    if (clip_coef != nullptr) scale *= *clip_coef;
    const int per = (g.n_vec + gridDim.x - 1) / gridDim.x;
    const int c0 = blockIdx.x * per;
    const int c1 = min(g.n_vec, c0 + per);
    float sumsq = 0.f;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    MgwCursor cur = mgw_cursor();
    for (int v0 = c0 + warp * 32 * U + lane; v0 < c1; v0 += blockDim.x * U) {
        float4 x[U];
        mgw_load_grad_batch<U>(g, v0, 32, c1, cur, scale, x);
        mgw_consume_batch<U>(g, v0, 32, c1, cur, x, mode, hyper, first_step, sumsq);
    }
    if (mode & MGW_MODE_SUMSQ) {
        float r = mgw_block_sum(sumsq, red);
        if (threadIdx.x == 0) sumsq_partials[blockIdx.x] = r;
    }
}

__global__ void mgw_clip_coef_kernel(const float* __restrict__ partials, int n, float max_norm, float* __restrict__ out2) {
    // single warp, fixed order: lane i sums partials i, i+32, ... then a fixed shuffle tree
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += 32) s += partials[i];
    for (int o = 16; o > 0; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) {
        const float norm = sqrtf(s);
        out2[0] = norm;
        const float c = max_norm / (norm + 1e-6f);
        out2[1] = c < 1.f ? c : 1.f;
    }
}

extern "C" int mgw_multi_tensor_sgd(const MgwGroup* group, const MgwHyper* hyper, const float* clip_coef, float grad_scale,
                                    int first_step, int mode, float* sumsq_partials, int n_ctas, void* stream) {
    if (group == nullptr || group->n_vec < 0 || n_ctas <= 0) return MGW_ERR_ARG;
    if ((mode & MGW_MODE_SUMSQ) && sumsq_partials == nullptr) return MGW_ERR_ARG;
    if (group->n_vec == 0) return MGW_OK;
    mgw_multi_tensor_sgd_kernel<2, 2><<<n_ctas, 512, 0, (cudaStream_t)stream>>>(*group, hyper, clip_coef, grad_scale, first_step,
                                                                                 mode, sumsq_partials);
    MGW_CUDA_CHECK(cudaGetLastError());
    return MGW_OK;
}

MGW_DEFINE_BOUNDS_READER(mgw_bounds_sgd)

extern "C" int mgw_group_sumsq(const MgwGroup* group, float* partials, int n_ctas, void* stream) {
    return mgw_multi_tensor_sgd(group, nullptr, nullptr, 1.f, 0, MGW_MODE_SUMSQ, partials, n_ctas, stream);
}

extern "C" int mgw_clip_coef(const float* partials, int n, float max_norm, float* out2, void* stream) {
    if (partials == nullptr || out2 == nullptr || n <= 0) return MGW_ERR_ARG;
    mgw_clip_coef_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(partials, n, max_norm, out2);
    MGW_CUDA_CHECK(cudaGetLastError());
    return MGW_OK;
}

// ---- allocation-free variant (declared in noalloc.h) ---------------------------------------------------
#include "noalloc.h"
#include <cstdio>

// Scratch for the per-CTA partial sums.  In host code this name is only a handle for
// cudaGetSymbolAddress(); the kernels receive the device address obtained from it.
static __device__ __align__(256) float g_static_partials[MGW_STATIC_MAX_PARTIALS];

namespace {
constexpr int kMaxDevices = 64;
// Device address of g_static_partials per device, filled on the first call on that device.  Atomic only so that two host
// threads making their first call at once both see a complete pointer (they would store the same value).  A
// cudaDeviceReset() invalidates the entry of that device; a process that resets a device must not call this afterwards.
std::atomic<float*> g_static_partials_addr[kMaxDevices];
}  // namespace

extern "C" int mgw_grad_clip_coef_static(const MgwGroup* group, float max_norm, float* out2, int n_ctas, void* stream) {
    if (group == nullptr || out2 == nullptr || group->n_vec < 0 || n_ctas < 1) return MGW_ERR_ARG;
    if (n_ctas > MGW_STATIC_MAX_PARTIALS) {
        static thread_local char msg[160];
        snprintf(msg, sizeof(msg), "n_ctas = %d exceeds the built-in scratch of %d partial sums", n_ctas, MGW_STATIC_MAX_PARTIALS);
        mgw_set_last_error(cudaErrorInvalidValue, msg, __FILE__, __LINE__);
        return MGW_ERR_TOO_LARGE;
    }
    int dev = -1;
    MGW_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return MGW_ERR_ARG;
    float* partials = g_static_partials_addr[dev].load(std::memory_order_acquire);
    if (partials == nullptr) {
        // once per device, with that device current: translate the symbol into this device's address
        MGW_CUDA_CHECK(cudaGetSymbolAddress((void**)&partials, g_static_partials));
        g_static_partials_addr[dev].store(partials, std::memory_order_release);
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (group->n_vec == 0) n_ctas = 1;
    mgw_multi_tensor_sgd_kernel<2, 2><<<n_ctas, 512, 0, s>>>(*group, nullptr, nullptr, 1.f, 0, MGW_MODE_SUMSQ, partials);
    MGW_CUDA_CHECK(cudaGetLastError());
    mgw_clip_coef_kernel<<<1, 32, 0, s>>>(partials, n_ctas, max_norm, out2);
    MGW_CUDA_CHECK(cudaGetLastError());
    return MGW_OK;
}
