// BatchNorm(+add)+ReLU for SMALL activations (at most 8192 rows, channels a multiple of 16, one resident wave of
// clusters): one kernel per direction instead of three.
//
// The three-launch kernels of bn_relu.cu are bandwidth-bound on large tensors, but on the 14x14 and 7x7 stages of a
// ResNet / DenseNet each launch takes 4-5 us for 1-3 us worth of data, and the tensor is read twice.  Here a
// thread-block CLUSTER of eight CTAs owns a slab of 16 channels: every CTA takes an eighth of the rows, a thread keeps its
// rows (up to R float4 values) in registers, the per-channel partial sums are combined through distributed shared
// memory in a fixed order after one cluster barrier, and the normalisation is applied to the values still in
// registers.  The hardware co-schedules the CTAs of a cluster, so the barrier needs no spin loop and cannot wait for a
// CTA that is not running.  One read of x, one write of y in the forward pass; backward keeps the masked gradient
// in registers and re-reads x, which the 126 MB L2 still holds.
//
// Thread layout of a CTA: 512 threads = 128 rows x 4 float4 lanes (16 channels, 64 bytes per row); a warp covers
// 8 rows.  Sums are reduced with a fixed shuffle tree inside the warp, across the 16 warps in warp order and across the
// 8 CTAs in rank order (in double), so results are reproducible run to run.
#include <cooperative_groups.h>

#include "api.h"

namespace cg = cooperative_groups;

namespace {

constexpr int kClusterSize = 8;
constexpr int kThreads = 512;
constexpr int kLanes = 4;                       // float4 lanes per row of a slab
constexpr int kSlab = 16;                       // channels per cluster
constexpr int kRowsPerPass = kThreads / kLanes; // 128
// Largest number of rows a thread holds.  Sixteen rows (a full register file per CTA, 128 CTAs for 256 channels) were
// measured equal or slower than the three-launch kernels inside a ResNet-50 step and are not built.
constexpr int kMaxRowsPerThread = 8;

struct Sums {
    float part[2][kSlab];       // this CTA's partial sums, read by the whole cluster
    float warp[16][2][kSlab];   // per-warp partials
    float tot[2][kSlab];        // cluster totals (identical in every CTA)
};

// Reduce (a, b) -- four channels per thread -- over all threads of the CTA that share the thread's lane; result in sm.part.
__device__ __forceinline__ void cta_reduce(float (&a)[4], float (&b)[4], Sums& sm) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tx = threadIdx.x & (kLanes - 1);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
#pragma unroll
        for (int o = 16; o >= kLanes; o >>= 1) {       // rows of the warp: lanes that differ in bits 2..4
            a[k] += __shfl_xor_sync(0xffffffffu, a[k], o);
            b[k] += __shfl_xor_sync(0xffffffffu, b[k], o);
        }
    }
    if (lane < kLanes) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            sm.warp[warp][0][tx * 4 + k] = a[k];
            sm.warp[warp][1][tx * 4 + k] = b[k];
        }
    }
    __syncthreads();
    if (threadIdx.x < 2 * kSlab) {
        const int which = threadIdx.x / kSlab, c = threadIdx.x % kSlab;
        float r = 0.f;
#pragma unroll
        for (int w = 0; w < 16; ++w) r += sm.warp[w][which][c];
        sm.part[which][c] = r;
    }
}

// After cta_reduce in every CTA of the cluster: totals of all eight CTAs into sm.tot (same values everywhere).
__device__ __forceinline__ void cluster_totals(cg::cluster_group& cluster, Sums& sm) {
    cluster.sync();                                                // every CTA's sm.part is written
    if (threadIdx.x < 2 * kSlab) {
        const int which = threadIdx.x / kSlab, c = threadIdx.x % kSlab;
        double r = 0.0;
        for (int rank = 0; rank < kClusterSize; ++rank) {
            const Sums* peer = cluster.map_shared_rank(&sm, rank);
            r += (double)peer->part[which][c];
        }
        sm.tot[which][c] = (float)r;
    }
    __syncthreads();
}

template <int R>
__global__ void __cluster_dims__(kClusterSize, 1, 1) __launch_bounds__(kThreads, 1)
bn_fwd_cluster_kernel(const float* __restrict__ x, const float* __restrict__ residual, float* __restrict__ y, int M, int C,
                      const float* __restrict__ gamma, const float* __restrict__ beta, float* running_mean, float* running_var,
                      long long* num_batches_tracked, float momentum, float eps, int relu, float* __restrict__ save_mean,
                      float* __restrict__ save_invstd, unsigned char* __restrict__ bits) {
    __shared__ Sums sm;
    __shared__ float sc_s[kSlab], sh_s[kSlab];
    cg::cluster_group cluster = cg::this_cluster();
    const int crank = (int)cluster.block_rank();
    const int slab = blockIdx.x / kClusterSize;
    const int tx = threadIdx.x & (kLanes - 1), ty = threadIdx.x >> 2;
    const int c0 = slab * kSlab + tx * 4;
    const int rows = (M + kClusterSize - 1) / kClusterSize;
    const int r0 = crank * rows, r1 = min(M, r0 + rows);

    float4 v[R];
    float s[4] = {0.f, 0.f, 0.f, 0.f}, q[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < R; ++k) {
        const int r = r0 + ty + k * kRowsPerPass;
        if (r < r1) {
            v[k] = *reinterpret_cast<const float4*>(x + (size_t)r * C + c0);
            s[0] += v[k].x; s[1] += v[k].y; s[2] += v[k].z; s[3] += v[k].w;
            q[0] = fmaf(v[k].x, v[k].x, q[0]); q[1] = fmaf(v[k].y, v[k].y, q[1]);
            q[2] = fmaf(v[k].z, v[k].z, q[2]); q[3] = fmaf(v[k].w, v[k].w, q[3]);
        }
    }
    cta_reduce(s, q, sm);
    cluster_totals(cluster, sm);
    if (threadIdx.x < kSlab) {
        const int c = slab * kSlab + threadIdx.x;
        const double mean = (double)sm.tot[0][threadIdx.x] / (double)M;
        double var = (double)sm.tot[1][threadIdx.x] / (double)M - mean * mean;
        if (var < 0.0) var = 0.0;
        const float istd = (float)(1.0 / sqrt(var + (double)eps));
        const float g = gamma ? gamma[c] : 1.f, b = beta ? beta[c] : 0.f;
        sc_s[threadIdx.x] = g * istd;
        sh_s[threadIdx.x] = b - (float)mean * (g * istd);
        if (crank == 0) {
            save_mean[c] = (float)mean;
            save_invstd[c] = istd;
            if (running_mean) {
                const double unbiased = M > 1 ? var * (double)M / (double)(M - 1) : var;
                running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * (float)mean;
                running_var[c] = (1.f - momentum) * running_var[c] + momentum * (float)unbiased;
            }
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0 && num_batches_tracked) *num_batches_tracked += 1;
    __syncthreads();
    const float sc[4] = {sc_s[tx * 4 + 0], sc_s[tx * 4 + 1], sc_s[tx * 4 + 2], sc_s[tx * 4 + 3]};
    const float sh[4] = {sh_s[tx * 4 + 0], sh_s[tx * 4 + 1], sh_s[tx * 4 + 2], sh_s[tx * 4 + 3]};
#pragma unroll
    for (int k = 0; k < R; ++k) {
        const int r = r0 + ty + k * kRowsPerPass;
        if (r < r1) {
            const size_t off = (size_t)r * C + c0;
            float4 o = make_float4(fmaf(v[k].x, sc[0], sh[0]), fmaf(v[k].y, sc[1], sh[1]), fmaf(v[k].z, sc[2], sh[2]),
                                   fmaf(v[k].w, sc[3], sh[3]));
            if (residual) {
                const float4 rr = *reinterpret_cast<const float4*>(residual + off);
                o.x += rr.x; o.y += rr.y; o.z += rr.z; o.w += rr.w;
            }
            if (bits)
                bits[off >> 2] = (unsigned char)((o.x > 0.f ? 1 : 0) | (o.y > 0.f ? 2 : 0) | (o.z > 0.f ? 4 : 0) | (o.w > 0.f ? 8 : 0));
            if (relu) { o.x = fmaxf(o.x, 0.f); o.y = fmaxf(o.y, 0.f); o.z = fmaxf(o.z, 0.f); o.w = fmaxf(o.w, 0.f); }
            *reinterpret_cast<float4*>(y + off) = o;
        }
    }
    cluster.sync();            // nobody leaves while a peer may still read its shared memory
}

// mask_mode as in bn_relu.cu: 0 none, 1 from the output y, 2 recomputed from x, 3 from the byte mask.
template <int R>
__global__ void __cluster_dims__(kClusterSize, 1, 1) __launch_bounds__(kThreads, 1)
bn_bwd_cluster_kernel(const float* __restrict__ dy, const float* __restrict__ dy2, const float* __restrict__ y,
                      const unsigned char* __restrict__ bits, const float* __restrict__ x, float* __restrict__ dz, float* __restrict__ dx,
                      int M, int C, const float* __restrict__ gamma, const float* __restrict__ beta,
                      const float* __restrict__ save_mean, const float* __restrict__ save_invstd, int mask_mode,
                      float* __restrict__ dgamma, float* __restrict__ dbeta) {
    __shared__ Sums sm;
    cg::cluster_group cluster = cg::this_cluster();
    const int crank = (int)cluster.block_rank();
    const int slab = blockIdx.x / kClusterSize;
    const int tx = threadIdx.x & (kLanes - 1), ty = threadIdx.x >> 2;
    const int c0 = slab * kSlab + tx * 4;
    const int rows = (M + kClusterSize - 1) / kClusterSize;
    const int r0 = crank * rows, r1 = min(M, r0 + rows);

    float mean[4], istd[4], sc[4], sh[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        mean[k] = save_mean[c0 + k];
        istd[k] = save_invstd[c0 + k];
        const float g = gamma ? gamma[c0 + k] : 1.f, b = beta ? beta[c0 + k] : 0.f;
        sc[k] = g * istd[k];
        sh[k] = b - mean[k] * sc[k];
    }
    float4 g[R];
    float s[4] = {0.f, 0.f, 0.f, 0.f}, q[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < R; ++k) {
        const int r = r0 + ty + k * kRowsPerPass;
        if (r < r1) {
            const size_t off = (size_t)r * C + c0;
            float4 gg = *reinterpret_cast<const float4*>(dy + off);
            const float4 xv = *reinterpret_cast<const float4*>(x + off);
            if (dy2) {
                const float4 h = *reinterpret_cast<const float4*>(dy2 + off);
                gg.x += h.x; gg.y += h.y; gg.z += h.z; gg.w += h.w;
            }
            if (mask_mode == 3) {
                const unsigned b = bits[off >> 2];
                gg.x = (b & 1u) ? gg.x : 0.f; gg.y = (b & 2u) ? gg.y : 0.f; gg.z = (b & 4u) ? gg.z : 0.f; gg.w = (b & 8u) ? gg.w : 0.f;
            } else if (mask_mode == 1) {
                const float4 yv = *reinterpret_cast<const float4*>(y + off);
                gg.x = yv.x > 0.f ? gg.x : 0.f; gg.y = yv.y > 0.f ? gg.y : 0.f; gg.z = yv.z > 0.f ? gg.z : 0.f; gg.w = yv.w > 0.f ? gg.w : 0.f;
            } else if (mask_mode == 2) {
                gg.x = fmaf(xv.x, sc[0], sh[0]) > 0.f ? gg.x : 0.f; gg.y = fmaf(xv.y, sc[1], sh[1]) > 0.f ? gg.y : 0.f;
                gg.z = fmaf(xv.z, sc[2], sh[2]) > 0.f ? gg.z : 0.f; gg.w = fmaf(xv.w, sc[3], sh[3]) > 0.f ? gg.w : 0.f;
            }
            g[k] = gg;
            s[0] += gg.x; s[1] += gg.y; s[2] += gg.z; s[3] += gg.w;
            q[0] = fmaf(gg.x, (xv.x - mean[0]) * istd[0], q[0]); q[1] = fmaf(gg.y, (xv.y - mean[1]) * istd[1], q[1]);
            q[2] = fmaf(gg.z, (xv.z - mean[2]) * istd[2], q[2]); q[3] = fmaf(gg.w, (xv.w - mean[3]) * istd[3], q[3]);
            if (dz) *reinterpret_cast<float4*>(dz + off) = gg;
        }
    }
    cta_reduce(s, q, sm);
    cluster_totals(cluster, sm);
    if (crank == 0 && threadIdx.x < kSlab) {
        dbeta[slab * kSlab + threadIdx.x] = sm.tot[0][threadIdx.x];
        dgamma[slab * kSlab + threadIdx.x] = sm.tot[1][threadIdx.x];
    }
    const float inv_m = 1.f / (float)M;
    float db[4], dg[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        db[k] = sm.tot[0][tx * 4 + k] * inv_m;
        dg[k] = sm.tot[1][tx * 4 + k] * inv_m;
    }
#pragma unroll
    for (int k = 0; k < R; ++k) {
        const int r = r0 + ty + k * kRowsPerPass;
        if (r < r1) {
            const size_t off = (size_t)r * C + c0;
            const float4 xv = *reinterpret_cast<const float4*>(x + off);         // second read: served by L2
            float4 o;
            o.x = sc[0] * (g[k].x - db[0] - (xv.x - mean[0]) * istd[0] * dg[0]);
            o.y = sc[1] * (g[k].y - db[1] - (xv.y - mean[1]) * istd[1] * dg[1]);
            o.z = sc[2] * (g[k].z - db[2] - (xv.z - mean[2]) * istd[2] * dg[2]);
            o.w = sc[3] * (g[k].w - db[3] - (xv.w - mean[3]) * istd[3] * dg[3]);
            *reinterpret_cast<float4*>(dx + off) = o;
        }
    }
    cluster.sync();
}

// Can the device place a cluster of the heaviest instantiations (most rows per thread)?  Asked once.
bool clusters_fit() {
    static const bool ok = [] {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(kClusterSize);
        cfg.blockDim = dim3(kThreads);
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = kClusterSize;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int nf = 0, nb = 0;
        if (cudaOccupancyMaxActiveClusters(&nf, bn_fwd_cluster_kernel<kMaxRowsPerThread>, &cfg) != cudaSuccess) { cudaGetLastError(); return false; }
        if (cudaOccupancyMaxActiveClusters(&nb, bn_bwd_cluster_kernel<kMaxRowsPerThread>, &cfg) != cudaSuccess) { cudaGetLastError(); return false; }
        return nf >= 1 && nb >= 1;
    }();
    return ok;
}

int rows_per_thread(long long M) {
    const long long per_cta = (M + kClusterSize - 1) / kClusterSize;
    return (int)((per_cta + kRowsPerPass - 1) / kRowsPerPass);
}

}  // namespace

extern "C" {

// 1 when the dispatcher should give an [M, C] problem to the cluster kernels on the current device: at most 8192 rows,
// C a multiple of 16 and at most 288 (one CTA per SM holds all clusters).  Measured inside training steps on B200:
// DenseNet-201's 128-channel layers (64 CTAs) gain 2-3 % of the step; 256 channels with 16 rows per thread (a full
// register file per CTA) and 512 channels (256 CTAs, two per SM) were equal or slower than the three-launch kernels, and
// 1024+ channels (several waves of clusters) clearly slower (51 MB: 88 us against 56 us).
int mgw_bn_cluster_supported(long long M, int C) {
    if (!(M > 0 && M <= (long long)kMaxRowsPerThread * kRowsPerPass * kClusterSize && C > 0 && C % kSlab == 0)) return 0;
    return ((C / kSlab) * kClusterSize <= 148 && clusters_fit()) ? 1 : 0;
}

int mgw_bn_relu_fwd_cluster(const float* x, const float* residual, float* y, long long M, int C, const float* gamma, const float* beta,
                            float* running_mean, float* running_var, long long* num_batches_tracked, float momentum, float eps,
                            int relu, float* save_mean, float* save_invstd, unsigned char* relu_bits, void* stream) {
    if (x == nullptr || y == nullptr || save_mean == nullptr || save_invstd == nullptr || !mgw_bn_cluster_supported(M, C)) return MGW_ERR_ARG;
    if (relu_bits != nullptr && !relu) return MGW_ERR_ARG;
    const dim3 grid((C / kSlab) * kClusterSize), block(kThreads);
    cudaStream_t s = (cudaStream_t)stream;
    const int R = rows_per_thread(M);
#define MGW_LAUNCH_FWD(RR)                                                                                                      \
    bn_fwd_cluster_kernel<RR><<<grid, block, 0, s>>>(x, residual, y, (int)M, C, gamma, beta, running_mean, running_var,          \
                                                     num_batches_tracked, momentum, eps, relu, save_mean, save_invstd, relu_bits)
    if (R <= 2) MGW_LAUNCH_FWD(2);
    else if (R <= 4) MGW_LAUNCH_FWD(4);
    else MGW_LAUNCH_FWD(8);
#undef MGW_LAUNCH_FWD
    MGW_CUDA_CHECK(cudaGetLastError());
    return MGW_OK;
}

int mgw_bn_relu_bwd_cluster(const float* dy, const float* dy2, const float* y, const float* x, float* dz, float* dx, long long M, int C,
                            const float* gamma, const float* beta, const float* save_mean, const float* save_invstd, int relu,
                            float* dgamma, float* dbeta, const unsigned char* relu_bits, void* stream) {
    if (dy == nullptr || x == nullptr || dx == nullptr || dgamma == nullptr || dbeta == nullptr || save_mean == nullptr ||
        save_invstd == nullptr || !mgw_bn_cluster_supported(M, C))
        return MGW_ERR_ARG;
    if (relu_bits != nullptr && !relu) return MGW_ERR_ARG;
    const int mask_mode = !relu ? 0 : (relu_bits != nullptr ? 3 : (y != nullptr ? 1 : 2));
    const dim3 grid((C / kSlab) * kClusterSize), block(kThreads);
    cudaStream_t s = (cudaStream_t)stream;
    const int R = rows_per_thread(M);
#define MGW_LAUNCH_BWD(RR)                                                                                                   \
    bn_bwd_cluster_kernel<RR><<<grid, block, 0, s>>>(dy, dy2, y, relu_bits, x, dz, dx, (int)M, C, gamma, beta, save_mean,      \
                                                     save_invstd, mask_mode, dgamma, dbeta)
    if (R <= 2) MGW_LAUNCH_BWD(2);
    else if (R <= 4) MGW_LAUNCH_BWD(4);
    else MGW_LAUNCH_BWD(8);
#undef MGW_LAUNCH_BWD
    MGW_CUDA_CHECK(cudaGetLastError());
    return MGW_OK;
}

}  // extern "C"
