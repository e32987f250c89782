// Fused training-mode BatchNorm (+ residual add) (+ ReLU), forward and backward, for activations
// stored as a dense [M, C] matrix with channels innermost: channels-last 4-D tensors
// (M = N*H*W) and 2-D inputs of BatchNorm1d (M = batch).
//
// Forward = two streaming passes instead of cuDNN BatchNorm + add + ReLU (two extra passes over the
// activation):
//   bn_stats_kernel        : per-channel sum / sum of squares, one deterministic partial per row split;
//                            the LAST block of a channel tile to finish combines the tile's partials in double,
//                            saves mean / inv-std and updates the running statistics (see "finalize" below)
//   bn_apply_kernel        : y = relu(x * scale + shift (+ residual))
// Backward:
//   bn_bwd_reduce_kernel   : dz = dy * relu'(.); partial sums of dz and dz * xhat; last block: dgamma, dbeta
//   bn_bwd_apply_kernel    : dx = scale * (dz - (dbeta + xhat * dgamma) / M)
// Finalize: every block of a channel tile bumps an arrival counter after its partials are visible; the block that
// sees the last count does the tile's (tiny) final reduction, in a fixed order, and resets the counter.  Nobody
// waits for anybody, so nothing can hang, and the result does not depend on which block came last.  That makes
// two launches per direction; on the 14x14 and 7x7 stages of a ResNet a separate finalize launch cost as much as
// the data movement itself.  Problems with very many row splits keep the separate bn_*_finalize_kernel (a single
// block would take longer over the partials than a launch costs).
// With a residual input dz is materialised (it is the residual's gradient) and the ReLU mask is read
// from the saved output; without one neither y nor dz is touched: the mask is recomputed from x, so
// the backward pass is 4 reads + 1 write of the activation instead of 5 + 2.
//
// Thread layout: a block is TX lanes along channels (each lane owns VEC consecutive channels, one
// 16-byte access when VEC = 4) by TY rows; grid.x tiles the channels, grid.y splits the rows.
// All of it is bandwidth-bound; the second pass of each direction re-reads tensors that the first
// pass just streamed, which the 126 MB L2 serves for the smaller layers.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include "api.h"

namespace {

constexpr int kThreads = 512;

// Programmatic dependent launch: the second and third kernel of a direction are launched with the "programmatic
// stream serialization" attribute, so their blocks may become resident while the previous kernel's last blocks
// are still running; they do their index arithmetic and then wait (griddepcontrol.wait) until the previous grid
// has completed and its writes are visible.  That removes the idle gap between the short kernels of the small
// layers.  Both instructions are no-ops in a kernel that was launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool env_on(const char* name, bool dflt) {
    const char* v = getenv(name);
    if (v == nullptr || *v == 0) return dflt;
    return !(v[0] == '0' || v[0] == 'f' || v[0] == 'F' || v[0] == 'n' || v[0] == 'N');
}

template <typename... KArgs, typename... Args>
cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool dependent, Args... args) {
    static const bool pdl = env_on("MGWFBP_BN_PDL", true);
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    const bool use = dependent && pdl;
    cfg.attrs = use ? attr : nullptr;
    cfg.numAttrs = use ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <int VEC> struct Vec;
template <> struct Vec<4> { using T = float4; };
template <> struct Vec<1> { using T = float; };

template <int VEC>
__device__ __forceinline__ void load_vec(const float* p, float (&v)[VEC]) {
    if (VEC == 4) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1 % VEC] = t.y; v[2 % VEC] = t.z; v[3 % VEC] = t.w;
    } else {
        v[0] = *p;
    }
}

template <int VEC>
__device__ __forceinline__ void store_vec(float* p, const float (&v)[VEC]) {
    if (VEC == 4) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1 % VEC], v[2 % VEC], v[3 % VEC]);
    } else {
        *p = v[0];
    }
}

struct Tiling {
    int tx, ty, grid_x, grid_y, rows_per_split;
};

// How many SMs the BatchNorm kernels size their single resident wave for.  The kernels are laid out as exactly one
// wave (4 or 2 blocks per SM); when a communication kernel holds some SMs beside them (one 512-thread CTA per SM, at
// most `overlap_ctas` of them), a grid sized for all SMs no longer fits and its last blocks run as a second wave, which
// doubles the kernel's time for an 11 % loss of SMs.  A multi-GPU job therefore lowers the budget by the CTAs its
// overlapped communication kernels may use (mgw_bn_set_sm_budget); the kernels are bandwidth bound and lose nothing
// measurable on the remaining SMs when they have the GPU to themselves.
std::atomic<int> g_sm_budget{0};

int sm_budget() {
    int v = g_sm_budget.load();
    if (v > 0) return v;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms < 1) sms = 148;
    g_sm_budget.store(sms);
    return sms;
}

Tiling make_tiling(long long M, int C, int vec, int blocks_per_sm = 4) {
    Tiling t;
    const int lanes = (C + vec - 1) / vec;
    int tx = 1;
    while (tx < lanes && tx < 32) tx <<= 1;
    t.tx = tx;
    t.ty = kThreads / tx;
    t.grid_x = (lanes + tx - 1) / tx;
    const int target_blocks = sm_budget() * blocks_per_sm;    // exactly one resident wave on the SMs this job may count on
    long long max_splits = (M + t.ty - 1) / t.ty;
    long long gy = (target_blocks + t.grid_x - 1) / t.grid_x;
    if (gy > max_splits) gy = max_splits;
    if (gy > 1024) gy = 1024;
    if (gy < 1) gy = 1;
    t.grid_y = (int)gy;
    long long rps = (M + gy - 1) / gy;
    rps = (rps + t.ty - 1) / t.ty * t.ty;
    t.rows_per_split = (int)rps;
    t.grid_y = (int)((M + rps - 1) / rps);
    return t;
}

// Sum `a` and `b` over the TY rows of the block in a fixed order; valid in threads with ty == 0.
template <int VEC>
__device__ __forceinline__ void block_reduce_rows(float (&a)[VEC], float (&b)[VEC], float* smem, int tx, int ty, int TX, int TY) {
    float* sa = smem;
    float* sb = smem + kThreads * VEC;
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
        sa[(ty * TX + tx) * VEC + k] = a[k];
        sb[(ty * TX + tx) * VEC + k] = b[k];
    }
    __syncthreads();
    if (ty == 0) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            float ra = 0.f, rb = 0.f;
            for (int r = 0; r < TY; ++r) {
                ra += sa[(r * TX + tx) * VEC + k];
                rb += sb[(r * TX + tx) * VEC + k];
            }
            a[k] = ra;
            b[k] = rb;
        }
    }
    __syncthreads();
}

// Arrival counters of the fused finalize: a ring of slots, all zero whenever no kernel is using them (the last
// block of a tile puts its slot back to zero).  A launch takes gridDim.x consecutive slots; the host hands out
// ranges round-robin, so launches that could overlap on the GPU (different streams) do not share slots unless
// kRing / gridDim.x other launches were issued in between.
constexpr int kRing = 16384;
constexpr int kFuseMaxSplits = 320;      // more row splits than this: separate finalize kernel
constexpr int kFuseMaxTiles = 256;
__device__ unsigned int g_bn_arrivals[kRing];

struct FwdFinal {
    float* running_mean; float* running_var; long long* num_batches_tracked;
    float momentum, eps;
    float* save_mean; float* save_invstd;
    int slot0;               // first arrival slot of this launch, or -1: a separate kernel finalizes
};

struct BwdFinal {
    float* dgamma; float* dbeta;
    int slot0;
};

// True in every thread of exactly one block per channel tile: the one whose arrival completed the tile.
__device__ __forceinline__ bool last_block_of_tile(int slot0, int* flag) {
    __threadfence();                         // this thread's partials are visible device-wide ...
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();                     // ... and so are those of the whole block, before the arrival is counted
        const unsigned prev = atomicAdd(&g_bn_arrivals[slot0 + blockIdx.x], 1u);
        *flag = (prev == gridDim.y - 1);
        __threadfence();
    }
    __syncthreads();
    return *flag != 0;
}

// Totals of ONE of the two partial arrays (which = 0 / 1) for the channels of this block's tile, combined in double
// in an order that depends only on the launch geometry.  CT (channels per tile) is a multiple of VEC; a thread owns VEC
// consecutive channels (one 16-byte load per partial row when VEC = 4) and every (512 * VEC / CT)-th partial row; the
// per-thread sums meet in shared memory and the first CT / VEC threads finish them.  Kept out of line: it runs in
// one block per tile only, and its registers must not weigh on the streaming loop of the kernel around it.
template <int VEC>
__device__ __noinline__ void tile_totals(const float* __restrict__ partials, int which, int n_splits, int C, int CT, double* sm,
                                         double (&a)[VEC]) {
    const int lanes = CT / VEC;
    const int lane = threadIdx.x % lanes, part = threadIdx.x / lanes, nparts = kThreads / lanes;
    const int c = blockIdx.x * CT + lane * VEC;
    double ra[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) ra[k] = 0.0;
    if (c < C) {
        const float* base = partials + (size_t)which * C + c;
#pragma unroll 4
        for (int s = part; s < n_splits; s += nparts) {
            const float* ps = base + (size_t)s * 2 * C;
            if (VEC == 4) {
                const float4 t0 = __ldcg(reinterpret_cast<const float4*>(ps));
                ra[0] += (double)t0.x; ra[1 % VEC] += (double)t0.y; ra[2 % VEC] += (double)t0.z; ra[3 % VEC] += (double)t0.w;
            } else {
                ra[0] += (double)__ldcg(ps);
            }
        }
    }
    __syncthreads();                         // the staging area is free (row reduction, or the previous array)
#pragma unroll
    for (int k = 0; k < VEC; ++k) sm[(part * lanes + lane) * VEC + k] = ra[k];
    __syncthreads();
#pragma unroll
    for (int k = 0; k < VEC; ++k) a[k] = 0.0;
    if (part == 0) {
        for (int r = 0; r < nparts; ++r) {
#pragma unroll
            for (int k = 0; k < VEC; ++k) a[k] += sm[(r * lanes + lane) * VEC + k];
        }
    }
}

__device__ __forceinline__ void fwd_finalize_channel(double sum, double sq, long long M, int c, const FwdFinal& f) {
    const double mean = sum / (double)M;
    double var = sq / (double)M - mean * mean;
    if (var < 0.0) var = 0.0;
    f.save_mean[c] = (float)mean;
    f.save_invstd[c] = (float)(1.0 / sqrt(var + (double)f.eps));
    if (f.running_mean) {
        const double unbiased = M > 1 ? var * (double)M / (double)(M - 1) : var;
        f.running_mean[c] = (1.f - f.momentum) * f.running_mean[c] + f.momentum * (float)mean;
        f.running_var[c] = (1.f - f.momentum) * f.running_var[c] + f.momentum * (float)unbiased;
    }
}

template <int VEC>
__global__ void __launch_bounds__(kThreads, 4)
bn_stats_kernel(const float* __restrict__ x, long long ldx, long long M, int C, int TX, int rows_per_split, float* __restrict__ partials,
                const FwdFinal fin) {
    extern __shared__ float smem[];
    pdl_release_dependents();
    const int TY = kThreads / TX;
    const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;
    const int c0 = (blockIdx.x * TX + tx) * VEC;
    const bool active = c0 < C;
    float s[VEC], q[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) s[k] = q[k] = 0.f;
    const long long r0 = (long long)blockIdx.y * rows_per_split;
    const long long r1 = min(M, r0 + rows_per_split);
    if (active) {
        for (long long r = r0 + ty; r < r1; r += TY) {
            float v[VEC];
            load_vec<VEC>(x + r * ldx + c0, v);
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                s[k] += v[k];
                q[k] = fmaf(v[k], v[k], q[k]);
            }
        }
    }
    block_reduce_rows<VEC>(s, q, smem, tx, ty, TX, TY);
    if (ty == 0 && active) {
        float* ps = partials + (size_t)blockIdx.y * 2 * C;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            if (c0 + k < C) {
                ps[c0 + k] = s[k];
                ps[C + c0 + k] = q[k];
            }
        }
    }
    if (fin.slot0 < 0) return;
    __shared__ int last;
    if (!last_block_of_tile(fin.slot0, &last)) return;
    double sum[VEC], sq[VEC];
    tile_totals<VEC>(partials, 0, gridDim.y, C, TX * VEC, reinterpret_cast<double*>(smem), sum);
    tile_totals<VEC>(partials, 1, gridDim.y, C, TX * VEC, reinterpret_cast<double*>(smem), sq);
    const int c = (blockIdx.x * TX + threadIdx.x) * VEC;
    if (threadIdx.x < TX) {
#pragma unroll
        for (int k = 0; k < VEC; ++k)
            if (c + k < C) fwd_finalize_channel(sum[k], sq[k], M, c + k, fin);
    }
    if (threadIdx.x == 0) {
        g_bn_arrivals[fin.slot0 + blockIdx.x] = 0u;
        if (blockIdx.x == 0 && fin.num_batches_tracked) *fin.num_batches_tracked += 1;
    }
}

// Sum the per-split partials of kFinCh channels per block: 128 lanes walk the partial rows (a few loads each), then two
// short shared-memory stages combine them in double, always in the same order.  Many small blocks instead of a few
// large ones: the kernel is pure latency (a handful of dependent loads), so what counts is how few of them are
// chained and how many SMs take part.  Valid in threads with lane == 0: totals of channel c.
constexpr int kFinCh = 8, kFinLanes = 128;

__device__ __forceinline__ void finalize_sums(const float* __restrict__ partials, int n_splits, int C, double& a, double& b, int& c,
                                              double (*sm)[kFinLanes][kFinCh], double (*sm2)[8][kFinCh]) {
    const int ch = threadIdx.x % kFinCh, lane = threadIdx.x / kFinCh;
    c = blockIdx.x * kFinCh + ch;
    double ra = 0.0, rb = 0.0;
    if (c < C) {
        for (int s = lane; s < n_splits; s += kFinLanes) {
            const float* ps = partials + (size_t)s * 2 * C;
            ra += (double)ps[c];
            rb += (double)ps[C + c];
        }
    }
    sm[0][lane][ch] = ra;
    sm[1][lane][ch] = rb;
    __syncthreads();
    if (lane < 8) {
        ra = rb = 0.0;
        for (int r = lane; r < kFinLanes; r += 8) {
            ra += sm[0][r][ch];
            rb += sm[1][r][ch];
        }
        sm2[0][lane][ch] = ra;
        sm2[1][lane][ch] = rb;
    }
    __syncthreads();
    a = b = 0.0;
    if (lane == 0) {
        for (int r = 0; r < 8; ++r) {
            a += sm2[0][r][ch];
            b += sm2[1][r][ch];
        }
    }
}

__global__ void __launch_bounds__(kFinCh * kFinLanes)
bn_fwd_finalize_kernel(const float* __restrict__ partials, int n_splits, long long M, int C, float* running_mean, float* running_var,
                       long long* num_batches_tracked, float momentum, float eps, float* __restrict__ save_mean,
                       float* __restrict__ save_invstd) {
    __shared__ double sm[2][kFinLanes][kFinCh];
    __shared__ double sm2[2][8][kFinCh];
    pdl_release_dependents();
    pdl_wait();
    double sum, sq;
    int c;
    finalize_sums(partials, n_splits, C, sum, sq, c, sm, sm2);
    if (threadIdx.x < kFinCh && c < C) {
        const FwdFinal f = {running_mean, running_var, num_batches_tracked, momentum, eps, save_mean, save_invstd, -1};
        fwd_finalize_channel(sum, sq, M, c, f);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0 && num_batches_tracked) *num_batches_tracked += 1;
}

__global__ void __launch_bounds__(kFinCh * kFinLanes)
bn_bwd_finalize_kernel(const float* __restrict__ partials, int n_splits, int C, float* __restrict__ dgamma, float* __restrict__ dbeta) {
    __shared__ double sm[2][kFinLanes][kFinCh];
    __shared__ double sm2[2][8][kFinCh];
    pdl_release_dependents();
    pdl_wait();
    double a, b;
    int c;
    finalize_sums(partials, n_splits, C, a, b, c, sm, sm2);
    if (threadIdx.x < kFinCh && c < C) {
        dbeta[c] = (float)a;
        dgamma[c] = (float)b;
    }
}

template <int VEC, bool BITS>
__global__ void __launch_bounds__(kThreads, 4)
bn_apply_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ residual, float* __restrict__ y, long long M, int C,
                int TX, int rows_per_split, const float* __restrict__ gamma, const float* __restrict__ beta, int relu,
                const float* __restrict__ save_mean, const float* __restrict__ save_invstd, unsigned char* __restrict__ bits) {
    pdl_wait();
    const int TY = kThreads / TX;
    const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;
    const int c0 = (blockIdx.x * TX + tx) * VEC;
    if (c0 >= C) return;
    float sc[VEC], sh[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
        const bool in = c0 + k < C;
        const float g = (in && gamma) ? gamma[c0 + k] : 1.f;
        const float b = (in && beta) ? beta[c0 + k] : 0.f;
        sc[k] = in ? g * save_invstd[c0 + k] : 0.f;
        sh[k] = in ? b - save_mean[c0 + k] * sc[k] : 0.f;
    }
    const long long r0 = (long long)blockIdx.y * rows_per_split;
    const long long r1 = min(M, r0 + rows_per_split);
    for (long long r = r0 + ty; r < r1; r += TY) {
        float v[VEC], o[VEC];
        load_vec<VEC>(x + r * ldx + c0, v);
        if (residual) {
            float rr[VEC];
            load_vec<VEC>(residual + r * C + c0, rr);
#pragma unroll
            for (int k = 0; k < VEC; ++k) o[k] = fmaf(v[k], sc[k], sh[k]) + rr[k];
        } else {
#pragma unroll
            for (int k = 0; k < VEC; ++k) o[k] = fmaf(v[k], sc[k], sh[k]);
        }
        if (VEC == 4 && BITS) {
            // which of the four outputs the ReLU lets through, one byte per float4: backward reads this
            // instead of the whole output tensor
            bits[(r * C + c0) >> 2] = (unsigned char)((o[0] > 0.f ? 1 : 0) | (o[1 % VEC] > 0.f ? 2 : 0) |
                                                      (o[2 % VEC] > 0.f ? 4 : 0) | (o[3 % VEC] > 0.f ? 8 : 0));
        }
        if (relu) {
#pragma unroll
            for (int k = 0; k < VEC; ++k) o[k] = fmaxf(o[k], 0.f);
        }
        store_vec<VEC>(y + r * C + c0, o);
    }
}

// Description of a 3x3 / stride 2 / pad 1 max-pool that follows the BatchNorm+ReLU (the ResNet / DenseNet
// stem).  When `dp` is set, the gradient of the (never materialised) ReLU output is gathered from the
// pooled gradient: an input position collects dp of the up-to-four windows whose arg-max it was.
struct PoolArgs {
    const float* dp;             // [N, OH, OW, C] gradient of the pooled output, or null
    const unsigned char* idx;    // [N, OH, OW, C] arg-max position inside the window (kh * 3 + kw)
    int H, W, OH, OW;
};

template <int VEC>
__device__ __forceinline__ void pooled_grad(float (&g)[VEC], const PoolArgs& pa, long long r, int c0, int C) {
    const int iw = (int)(r % pa.W);
    const long long t = r / pa.W;
    const int ih = (int)(t % pa.H);
    const long long n = t / pa.H;
#pragma unroll
    for (int k = 0; k < VEC; ++k) g[k] = 0.f;
    const int oh0 = ih >> 1, oh1 = min(pa.OH - 1, (ih + 1) >> 1);
    const int ow0 = iw >> 1, ow1 = min(pa.OW - 1, (iw + 1) >> 1);
    for (int oh = oh0; oh <= oh1; ++oh) {
        const int kh = ih - (2 * oh - 1);
        for (int ow = ow0; ow <= ow1; ++ow) {
            const int code = kh * 3 + (iw - (2 * ow - 1));
            const size_t o = (((size_t)n * pa.OH + oh) * pa.OW + ow) * C + c0;
            float d[VEC];
            load_vec<VEC>(pa.dp + o, d);
            if (VEC == 4) {
                const uchar4 m = *reinterpret_cast<const uchar4*>(pa.idx + o);
                if (m.x == code) g[0] += d[0];
                if (m.y == code) g[1 % VEC] += d[1 % VEC];
                if (m.z == code) g[2 % VEC] += d[2 % VEC];
                if (m.w == code) g[3 % VEC] += d[3 % VEC];
            } else {
                if (pa.idx[o] == code) g[0] += d[0];
            }
        }
    }
}

// Gradient entering the normalisation for one vector of channels: dy, masked by the ReLU.
// mask_mode 0: no ReLU; 1: mask from the saved output y; 2: mask recomputed from x (bitwise the same
// fused multiply-add as the forward pass, so the sign test agrees with what the forward pass clipped);
// 3: mask from the byte the forward pass stored for this float4 (y_row then points at that byte).
template <int VEC, bool BYTE_MASK = false>
__device__ __forceinline__ void masked_grad(float (&g)[VEC], const float (&xv)[VEC], const float* __restrict__ y_row, int mask_mode,
                                            const float (&sc)[VEC], const float (&sh)[VEC]) {
    if (BYTE_MASK && mask_mode == 3) {
        const unsigned b = *reinterpret_cast<const unsigned char*>(y_row);
#pragma unroll
        for (int k = 0; k < VEC; ++k) g[k] = ((b >> k) & 1u) ? g[k] : 0.f;
    } else if (mask_mode == 1) {
        float yv[VEC];
        load_vec<VEC>(y_row, yv);
#pragma unroll
        for (int k = 0; k < VEC; ++k) g[k] = yv[k] > 0.f ? g[k] : 0.f;
    } else if (mask_mode == 2) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) g[k] = fmaf(xv[k], sc[k], sh[k]) > 0.f ? g[k] : 0.f;
    }
}

template <int VEC>
__device__ __forceinline__ void load_channel_consts(int c0, int C, const float* __restrict__ gamma, const float* __restrict__ beta,
                                                    const float* __restrict__ save_mean, const float* __restrict__ save_invstd,
                                                    float (&mean)[VEC], float (&istd)[VEC], float (&sc)[VEC], float (&sh)[VEC]) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
        const bool in = c0 + k < C;
        mean[k] = in ? save_mean[c0 + k] : 0.f;
        istd[k] = in ? save_invstd[c0 + k] : 0.f;
        const float g = (in && gamma) ? gamma[c0 + k] : 1.f;
        const float b = (in && beta) ? beta[c0 + k] : 0.f;
        sc[k] = in ? g * istd[k] : 0.f;
        sh[k] = in ? b - mean[k] * sc[k] : 0.f;
    }
}

template <int VEC, bool POOL>
__global__ void __launch_bounds__(kThreads, 2)
bn_bwd_reduce_kernel(const float* __restrict__ dy, const float* __restrict__ dy2, const float* __restrict__ y,
                     const unsigned char* __restrict__ bits, const float* __restrict__ x, long long ldx, float* __restrict__ dz,
                     long long M, int C, int TX, int rows_per_split, const float* __restrict__ gamma, const float* __restrict__ beta,
                     const float* __restrict__ save_mean, const float* __restrict__ save_invstd, int mask_mode,
                     float* __restrict__ partials, const PoolArgs pool, const BwdFinal fin) {
    extern __shared__ float smem[];
    pdl_release_dependents();
    const int TY = kThreads / TX;
    const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;
    const int c0 = (blockIdx.x * TX + tx) * VEC;
    const bool active = c0 < C;
    float s[VEC], q[VEC], mean[VEC], istd[VEC], sc[VEC], sh[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) s[k] = q[k] = 0.f;
    load_channel_consts<VEC>(active ? c0 : C, C, gamma, beta, save_mean, save_invstd, mean, istd, sc, sh);
    const long long r0 = (long long)blockIdx.y * rows_per_split;
    const long long r1 = min(M, r0 + rows_per_split);
    if (active) {
        long long r = r0 + ty;
        for (; r < r1; r += TY) {
            float g[VEC], xv[VEC];
            if (POOL) pooled_grad<VEC>(g, pool, r, c0, C); else load_vec<VEC>(dy + r * C + c0, g);
            load_vec<VEC>(x + r * ldx + c0, xv);
            if (dy2) {
                float h[VEC];
                load_vec<VEC>(dy2 + r * C + c0, h);
#pragma unroll
                for (int k = 0; k < VEC; ++k) g[k] += h[k];
            }
            masked_grad<VEC, true>(g, xv, mask_mode == 1 ? y + r * C + c0
                                                     : (mask_mode == 3 ? reinterpret_cast<const float*>(bits + ((r * C + c0) >> 2)) : nullptr),
                                   mask_mode, sc, sh);
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                s[k] += g[k];
                q[k] = fmaf(g[k], (xv[k] - mean[k]) * istd[k], q[k]);
            }
            if (dz) store_vec<VEC>(dz + r * C + c0, g);
        }
    }
    block_reduce_rows<VEC>(s, q, smem, tx, ty, TX, TY);
    if (ty == 0 && active) {
        float* ps = partials + (size_t)blockIdx.y * 2 * C;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            if (c0 + k < C) {
                ps[c0 + k] = s[k];
                ps[C + c0 + k] = q[k];
            }
        }
    }
    if (fin.slot0 < 0) return;
    __shared__ int last;
    if (!last_block_of_tile(fin.slot0, &last)) return;
    double a[VEC], b[VEC];
    tile_totals<VEC>(partials, 0, gridDim.y, C, TX * VEC, reinterpret_cast<double*>(smem), a);
    tile_totals<VEC>(partials, 1, gridDim.y, C, TX * VEC, reinterpret_cast<double*>(smem), b);
    const int c = (blockIdx.x * TX + threadIdx.x) * VEC;
    if (threadIdx.x < TX) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            if (c + k < C) {
                fin.dbeta[c + k] = (float)a[k];
                fin.dgamma[c + k] = (float)b[k];
            }
        }
    }
    if (threadIdx.x == 0) g_bn_arrivals[fin.slot0 + blockIdx.x] = 0u;
}

// gsrc is dz (mask already applied, mask_mode 0) or dy (mask applied here again, mask_mode 1 / 2).
template <int VEC, bool POOL>
__global__ void __launch_bounds__(kThreads, 2)
bn_bwd_apply_kernel(const float* __restrict__ gsrc, const float* __restrict__ gsrc2, const float* __restrict__ y, const float* __restrict__ x,
                    long long ldx, float* __restrict__ dx, long long lddx, int accumulate,
                    long long M, int C, int TX, int rows_per_split, const float* __restrict__ gamma, const float* __restrict__ beta,
                    const float* __restrict__ save_mean, const float* __restrict__ save_invstd, int mask_mode,
                    const float* __restrict__ dgamma, const float* __restrict__ dbeta, const PoolArgs pool) {
    pdl_wait();
    const int TY = kThreads / TX;
    const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;
    const int c0 = (blockIdx.x * TX + tx) * VEC;
    if (c0 >= C) return;
    const float inv_m = 1.f / (float)M;
    float mean[VEC], istd[VEC], sc[VEC], sh[VEC], db[VEC], dg[VEC];
    load_channel_consts<VEC>(c0, C, gamma, beta, save_mean, save_invstd, mean, istd, sc, sh);
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
        const bool in = c0 + k < C;
        db[k] = in ? dbeta[c0 + k] * inv_m : 0.f;
        dg[k] = in ? dgamma[c0 + k] * inv_m : 0.f;
    }
    const long long r0 = (long long)blockIdx.y * rows_per_split;
    const long long r1 = min(M, r0 + rows_per_split);
    for (long long r = r0 + ty; r < r1; r += TY) {
        float g[VEC], xv[VEC], o[VEC];
        if (POOL) pooled_grad<VEC>(g, pool, r, c0, C); else load_vec<VEC>(gsrc + r * C + c0, g);
        load_vec<VEC>(x + r * ldx + c0, xv);
        if (gsrc2) {
            float h[VEC];
            load_vec<VEC>(gsrc2 + r * C + c0, h);
#pragma unroll
            for (int k = 0; k < VEC; ++k) g[k] += h[k];
        }
        masked_grad<VEC>(g, xv, mask_mode == 1 ? y + r * C + c0 : nullptr, mask_mode, sc, sh);
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            const float xhat = (xv[k] - mean[k]) * istd[k];
            o[k] = sc[k] * (g[k] - db[k] - xhat * dg[k]);
        }
        float* dst = dx + r * lddx + c0;
        if (accumulate) {
            // the input gradient joins what other consumers of the same tensor have already added at dst (a dense block's
            // gradient buffer): one read-modify-write here instead of a store plus a separate addition kernel
            float prev[VEC];
            load_vec<VEC>(dst, prev);
#pragma unroll
            for (int k = 0; k < VEC; ++k) o[k] = __fadd_rn(prev[k], o[k]);      // a separate rounding, as a separate kernel would do
        }
        store_vec<VEC>(dst, o);
    }
}

// y_pool = maxpool3x3/s2/p1(relu(x * scale + shift)) in one pass over x; the full-resolution ReLU output is
// never written.  One thread per (output pixel, 4 channels); idx records which of the nine taps won.
template <int VEC>
__global__ void __launch_bounds__(256)
bn_relu_maxpool_kernel(const float* __restrict__ x, float* __restrict__ yp, unsigned char* __restrict__ idx, int N, int H, int W,
                       int OH, int OW, int C, const float* __restrict__ gamma, const float* __restrict__ beta,
                       const float* __restrict__ save_mean, const float* __restrict__ save_invstd) {
    pdl_wait();
    const int lanes = C / VEC;
    const long long total = (long long)N * OH * OW * lanes;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c0 = (int)(i % lanes) * VEC;
        long long t = i / lanes;
        const int ow = (int)(t % OW); t /= OW;
        const int oh = (int)(t % OH);
        const long long n = t / OH;
        float mean[VEC], istd[VEC], sc[VEC], sh[VEC], best[VEC];
        int code[VEC];
        load_channel_consts<VEC>(c0, C, gamma, beta, save_mean, save_invstd, mean, istd, sc, sh);
#pragma unroll
        for (int k = 0; k < VEC; ++k) { best[k] = -INFINITY; code[k] = 0; }
#pragma unroll
        for (int kh = 0; kh < 3; ++kh) {
            const int ih = 2 * oh - 1 + kh;
            if (ih < 0 || ih >= H) continue;
#pragma unroll
            for (int kw = 0; kw < 3; ++kw) {
                const int iw = 2 * ow - 1 + kw;
                if (iw < 0 || iw >= W) continue;
                float v[VEC];
                load_vec<VEC>(x + (((size_t)n * H + ih) * W + iw) * C + c0, v);
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    const float z = fmaxf(fmaf(v[k], sc[k], sh[k]), 0.f);
                    if (z > best[k]) { best[k] = z; code[k] = kh * 3 + kw; }
                }
            }
        }
        const size_t o = (((size_t)n * OH + oh) * OW + ow) * C + c0;
        store_vec<VEC>(yp + o, best);
        if (VEC == 4) {
            *reinterpret_cast<uchar4*>(idx + o) = make_uchar4((unsigned char)code[0], (unsigned char)code[1 % VEC],
                                                              (unsigned char)code[2 % VEC], (unsigned char)code[3 % VEC]);
        } else {
            idx[o] = (unsigned char)code[0];
        }
    }
}

bool fuse_enabled() {
    static const bool fuse = env_on("MGWFBP_BN_FUSE_FINALIZE", false);
    return fuse;
}

bool fused_geometry(int gx, int gy) { return fuse_enabled() && gy <= kFuseMaxSplits && gx <= kFuseMaxTiles; }

// Arrival slots for a launch of grid (gx, gy), or -1 when the problem keeps the separate finalize kernel.
int take_slots(int gx, int gy) {
    static std::atomic<unsigned> next{0};
    if (!fused_geometry(gx, gy)) return -1;
    for (;;) {
        const unsigned off = next.fetch_add((unsigned)gx) % (unsigned)kRing;
        if (off + (unsigned)gx <= (unsigned)kRing) return (int)off;
    }
}

size_t reduce_smem(int vec) {
    const size_t rows = sizeof(float) * 2 * kThreads * vec, fin = sizeof(double) * kThreads * vec;
    return rows > fin ? rows : fin;
}

struct FwdArgs {
    const float* x; const float* residual; float* y; long long M; int C;
    const float* gamma; const float* beta; float* running_mean; float* running_var; long long* nbt;
    float momentum, eps; int relu; float* save_mean; float* save_invstd; float* partials; unsigned char* bits;
    long long ldx;       // floats between consecutive rows of x (>= C; x may be a channel slice of a wider tensor)
};

// statistics (+ finalize); returns the tiling for the caller's second pass
template <int VEC>
cudaError_t launch_stats(const FwdArgs& a, const Tiling& t, cudaStream_t s) {
    const dim3 grid(t.grid_x, t.grid_y), block(kThreads);
    const FwdFinal fin = {a.running_mean, a.running_var, a.nbt, a.momentum, a.eps, a.save_mean, a.save_invstd,
                          take_slots(t.grid_x, t.grid_y)};
    cudaError_t e = launch(bn_stats_kernel<VEC>, grid, block, reduce_smem(VEC), s, false, a.x, a.ldx, a.M, a.C, t.tx, t.rows_per_split,
                           a.partials, fin);
    if (e == cudaSuccess && fin.slot0 < 0)
        e = launch(bn_fwd_finalize_kernel, dim3((a.C + kFinCh - 1) / kFinCh), dim3(kFinCh * kFinLanes), 0, s, true, (const float*)a.partials, t.grid_y, a.M,
                   a.C, a.running_mean, a.running_var, a.nbt, a.momentum, a.eps, a.save_mean, a.save_invstd);
    return e;
}

template <int VEC>
cudaError_t launch_fwd(const FwdArgs& a, cudaStream_t s) {
    const Tiling t = make_tiling(a.M, a.C, VEC);
    cudaError_t e = launch_stats<VEC>(a, t, s);
    if (e != cudaSuccess) return e;
    const dim3 grid(t.grid_x, t.grid_y), block(kThreads);
    if (VEC == 4 && a.bits)
        return launch(bn_apply_kernel<VEC, true>, grid, block, 0, s, true, a.x, a.ldx, a.residual, a.y, a.M, a.C, t.tx, t.rows_per_split,
                      a.gamma, a.beta, a.relu, (const float*)a.save_mean, (const float*)a.save_invstd, a.bits);
    return launch(bn_apply_kernel<VEC, false>, grid, block, 0, s, true, a.x, a.ldx, a.residual, a.y, a.M, a.C, t.tx, t.rows_per_split,
                  a.gamma, a.beta, a.relu, (const float*)a.save_mean, (const float*)a.save_invstd, (unsigned char*)nullptr);
}

struct BwdArgs {
    const float* dy; const float* dy2; const float* y; const unsigned char* bits; const float* x; float* dz; float* dx;
    long long M; int C; const float* gamma; const float* beta; const float* save_mean; const float* save_invstd;
    int mask1, mask2; float* dgamma; float* dbeta; float* partials; PoolArgs pool;
    long long ldx;       // floats between consecutive rows of x (>= C)
    long long lddx;      // floats between consecutive rows of dx (>= C)
    int accumulate;      // dx += result instead of dx = result
};

template <int VEC, bool POOL>
cudaError_t launch_bwd(const BwdArgs& a, cudaStream_t s) {
    const Tiling t = make_tiling(a.M, a.C, VEC, 2);      // backward kernels hold 2 blocks per SM
    const dim3 grid(t.grid_x, t.grid_y), block(kThreads);
    const BwdFinal fin = {a.dgamma, a.dbeta, take_slots(t.grid_x, t.grid_y)};
    cudaError_t e = launch(bn_bwd_reduce_kernel<VEC, POOL>, grid, block, reduce_smem(VEC), s, false, a.dy, a.dy2, a.y, a.bits, a.x,
                           a.ldx, a.dz, a.M, a.C, t.tx, t.rows_per_split, a.gamma, a.beta, a.save_mean, a.save_invstd, a.mask1, a.partials,
                           a.pool, fin);
    if (e == cudaSuccess && fin.slot0 < 0)
        e = launch(bn_bwd_finalize_kernel, dim3((a.C + kFinCh - 1) / kFinCh), dim3(kFinCh * kFinLanes), 0, s, true, (const float*)a.partials, t.grid_y, a.C,
                   a.dgamma, a.dbeta);
    if (e != cudaSuccess) return e;
    const float* gsrc = a.dz != nullptr ? a.dz : a.dy;
    const float* gsrc2 = a.dz != nullptr ? nullptr : a.dy2;        // dz already holds the sum of both gradients
    return launch(bn_bwd_apply_kernel<VEC, POOL>, grid, block, 0, s, true, gsrc, gsrc2, a.y, a.x, a.ldx, a.dx, a.lddx, a.accumulate, a.M, a.C, t.tx,
                  t.rows_per_split, a.gamma, a.beta, a.save_mean, a.save_invstd, a.mask2, (const float*)a.dgamma,
                  (const float*)a.dbeta, a.pool);
}

}  // namespace

extern "C" {

// SMs the BatchNorm grids are sized for from now on (0: all SMs of the current device); returns the previous value.
// Set it before a training step is captured in a CUDA graph: grids are part of the capture.
int mgw_bn_set_sm_budget(int sms) {
    const int prev = sm_budget();
    int dev = 0, all = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&all, cudaDevAttrMultiProcessorCount, dev);
    g_sm_budget.store(sms <= 0 ? all : (sms > all ? all : sms));
    return prev;
}

// Number of floats the caller must provide in `partials` for an [M, C] problem.
size_t mgw_bn_partials_floats(long long M, int C) {
    const Tiling t = make_tiling(M, C, (C % 4 == 0) ? 4 : 1);
    return (size_t)t.grid_y * 2 * (size_t)C;
}

// Kernel launches one forward (backward = 0) or backward (backward = 1) call issues for an [M, C] problem:
// two when the finalize step rides in the reduction kernel, three otherwise.  (Reporting only.)
int mgw_bn_launches(long long M, int C, int backward) {
    const Tiling t = make_tiling(M, C, (C % 4 == 0) ? 4 : 1, backward ? 2 : 4);
    return fused_geometry(t.grid_x, t.grid_y) ? 2 : 3;
}

// ldx: floats between consecutive rows of x (>= C).  With ldx > C the input is a channel slice of a wider channels-last
// tensor (the first C channels of a DenseNet block buffer) and is read in place; y, residual and the mask stay dense.
// The 16-byte loads of the C % 4 == 0 path need ldx % 4 == 0 as well.
int mgw_bn_relu_fwd_ld(const float* x, long long ldx, const float* residual, float* y, long long M, int C, const float* gamma,
                       const float* beta, float* running_mean, float* running_var, long long* num_batches_tracked, float momentum,
                       float eps, int relu, float* save_mean, float* save_invstd, float* partials, unsigned char* relu_bits,
                       void* stream) {
    if (x == nullptr || y == nullptr || M <= 0 || C <= 0 || save_mean == nullptr || save_invstd == nullptr || partials == nullptr)
        return MGW_ERR_ARG;
    if (ldx < C || (C % 4 == 0 && ldx % 4 != 0)) return MGW_ERR_ARG;
    if (relu_bits != nullptr && (C % 4 != 0 || !relu)) return MGW_ERR_ARG;
    const FwdArgs a = {x, residual, y, M, C, gamma, beta, running_mean, running_var, num_batches_tracked, momentum, eps, relu,
                       save_mean, save_invstd, partials, relu_bits, ldx};
    MGW_CUDA_CHECK((C % 4 == 0) ? launch_fwd<4>(a, (cudaStream_t)stream) : launch_fwd<1>(a, (cudaStream_t)stream));
    return MGW_OK;
}

int mgw_bn_relu_fwd(const float* x, const float* residual, float* y, long long M, int C, const float* gamma, const float* beta,
                    float* running_mean, float* running_var, long long* num_batches_tracked, float momentum, float eps,
                    int relu, float* save_mean, float* save_invstd, float* partials, unsigned char* relu_bits, void* stream) {
    return mgw_bn_relu_fwd_ld(x, C, residual, y, M, C, gamma, beta, running_mean, running_var, num_batches_tracked, momentum, eps, relu,
                              save_mean, save_invstd, partials, relu_bits, stream);
}

// Backward.  dy2 (may be null) is a second incoming gradient of the same output -- a block output that feeds
// both the next convolution and the next shortcut -- and is added on load, which replaces autograd's separate
// add kernel.  With dz != null the masked gradient dy * (y > 0) is written there (it is also the gradient
// of the residual input) and the ReLU mask comes from y; dx may alias dz.  With dz == null nothing is
// materialised: both passes read dy and x and rebuild the mask from x (gamma / beta must be the forward
// values), which saves one read and one write of the activation.  relu_bits (may be null; needs C % 4 == 0)
// is the byte-per-float4 ReLU mask the forward pass recorded: with it the reduce pass reads M*C/4 bytes
// instead of the M*C floats of y.
// lddx / accumulate: dx has rows lddx floats apart (>= C) and, with accumulate != 0, receives dx += result: the layer's
// input gradient is added straight into a wider gradient buffer that other consumers of the same input add to as well
// (not together with dz: a residual branch needs the gradient itself).
int mgw_bn_relu_bwd_ld(const float* dy, const float* dy2, const float* y, const float* x, long long ldx, float* dz, float* dx,
                       long long lddx, int accumulate, long long M, int C, const float* gamma, const float* beta, const float* save_mean, const float* save_invstd, int relu,
                       float* dgamma, float* dbeta, float* partials, const unsigned char* relu_bits, void* stream) {
    if (dy == nullptr || x == nullptr || dx == nullptr || M <= 0 || C <= 0 || partials == nullptr) return MGW_ERR_ARG;
    if (ldx < C || (C % 4 == 0 && ldx % 4 != 0)) return MGW_ERR_ARG;
    if (lddx < C || (C % 4 == 0 && lddx % 4 != 0) || ((accumulate || lddx != C) && dz != nullptr)) return MGW_ERR_ARG;
    // the byte mask serves the reduce pass; the apply pass then reads the masked gradient dz, which must exist
    if (relu_bits != nullptr && (C % 4 != 0 || !relu || dz == nullptr)) return MGW_ERR_ARG;
    if (dgamma == nullptr || dbeta == nullptr || save_mean == nullptr || save_invstd == nullptr) return MGW_ERR_ARG;
    const int mask1 = !relu ? 0 : (relu_bits != nullptr ? 3 : (y != nullptr ? 1 : 2));          // mask used by the reduce pass
    const int mask2 = dz != nullptr ? 0 : mask1;                   // apply pass: dz already carries the mask
    const BwdArgs a = {dy, dy2, y, relu_bits, x, dz, dx, M, C, gamma, beta, save_mean, save_invstd, mask1, mask2, dgamma, dbeta,
                       partials, {nullptr, nullptr, 0, 0, 0, 0}, ldx, lddx, accumulate};
    const cudaError_t e = (C % 4 == 0) ? launch_bwd<4, false>(a, (cudaStream_t)stream) : launch_bwd<1, false>(a, (cudaStream_t)stream);
    MGW_CUDA_CHECK(e);
    return MGW_OK;
}

// The same with x dense (ldx = C).
int mgw_bn_relu_bwd(const float* dy, const float* dy2, const float* y, const float* x, float* dz, float* dx, long long M, int C, const float* gamma,
                    const float* beta, const float* save_mean, const float* save_invstd, int relu, float* dgamma, float* dbeta,
                    float* partials, const unsigned char* relu_bits, void* stream) {
    return mgw_bn_relu_bwd_ld(dy, dy2, y, x, C, dz, dx, C, 0, M, C, gamma, beta, save_mean, save_invstd, relu, dgamma, dbeta, partials,
                              relu_bits, stream);
}

// BatchNorm + ReLU + 3x3/stride-2/pad-1 max-pool of a channels-last [N, H, W, C] tensor (the ResNet / DenseNet stem).
// Statistics over x as usual; the normalised full-resolution tensor is never written: the second pass pools
// on the fly and stores [N, OH, OW, C] values plus one byte per value naming the winning tap.
int mgw_bn_relu_maxpool_fwd(const float* x, float* y_pool, unsigned char* idx, int N, int H, int W, int C, const float* gamma,
                            const float* beta, float* running_mean, float* running_var, long long* num_batches_tracked,
                            float momentum, float eps, float* save_mean, float* save_invstd, float* partials, void* stream) {
    if (x == nullptr || y_pool == nullptr || idx == nullptr || N <= 0 || H <= 0 || W <= 0 || C <= 0 || partials == nullptr) return MGW_ERR_ARG;
    const long long M = (long long)N * H * W;
    const int OH = (H + 2 - 3) / 2 + 1, OW = (W + 2 - 3) / 2 + 1;
    const int vec = (C % 4 == 0) ? 4 : 1;
    const Tiling t = make_tiling(M, C, vec);
    cudaStream_t s = (cudaStream_t)stream;
    const long long work = (long long)N * OH * OW * (C / vec);
    const int pgrid = (int)((work + 255) / 256 < 148LL * 16 ? (work + 255) / 256 : 148LL * 16);
    const FwdArgs a = {x, nullptr, nullptr, M, C, gamma, beta, running_mean, running_var, num_batches_tracked, momentum, eps, 1,
                       save_mean, save_invstd, partials, nullptr, C};
    if (vec == 4) {
        MGW_CUDA_CHECK(launch_stats<4>(a, t, s));
        MGW_CUDA_CHECK(launch(bn_relu_maxpool_kernel<4>, dim3(pgrid), dim3(256), 0, s, true, x, y_pool, idx, N, H, W, OH, OW, C, gamma,
                              beta, (const float*)save_mean, (const float*)save_invstd));
    } else {
        MGW_CUDA_CHECK(launch_stats<1>(a, t, s));
        MGW_CUDA_CHECK(launch(bn_relu_maxpool_kernel<1>, dim3(pgrid), dim3(256), 0, s, true, x, y_pool, idx, N, H, W, OH, OW, C, gamma,
                              beta, (const float*)save_mean, (const float*)save_invstd));
    }
    return MGW_OK;
}

// Backward of the above: dp is the gradient of the pooled output; the gradient of the un-pooled ReLU output is
// gathered from dp / idx inside both BatchNorm passes (never materialised), the ReLU mask is rebuilt from x.
int mgw_bn_relu_maxpool_bwd(const float* dp, const unsigned char* idx, const float* x, float* dx, int N, int H, int W, int C,
                            const float* gamma, const float* beta, const float* save_mean, const float* save_invstd,
                            float* dgamma, float* dbeta, float* partials, void* stream) {
    if (dp == nullptr || idx == nullptr || x == nullptr || dx == nullptr || partials == nullptr || dgamma == nullptr || dbeta == nullptr)
        return MGW_ERR_ARG;
    const long long M = (long long)N * H * W;
    const BwdArgs a = {nullptr, nullptr, nullptr, nullptr, x, nullptr, dx, M, C, gamma, beta, save_mean, save_invstd, 2, 2, dgamma,
                       dbeta, partials, {dp, idx, H, W, (H + 2 - 3) / 2 + 1, (W + 2 - 3) / 2 + 1}, C, C, 0};
    const cudaError_t e = (C % 4 == 0) ? launch_bwd<4, true>(a, (cudaStream_t)stream) : launch_bwd<1, true>(a, (cudaStream_t)stream);
    MGW_CUDA_CHECK(e);
    return MGW_OK;
}

}  // extern "C"
