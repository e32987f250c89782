// Fused gradient all-reduce for one merged group, launched from the backward hook of the group's
// last tensor on a side stream:
//
//   pack (gather the group's scattered gradient tensors through a pointer table)
//   -> sum across GPUs through peer memory (NVLink 5 / NVSwitch loads and stores, or NVLS multimem)
//   -> x 1/N
//   -> weight decay + momentum + learning-rate update of the parameters (optional)
//   -> averaged gradient written back / sum of squares emitted (optional)
//
// in ONE kernel.  No NCCL call and no separate elementwise kernel runs on this path.
//
// Work split: CTA b owns a contiguous chunk of the group's float4 slots and only ever talks to CTA
// b of the other ranks, through its own row of flags, so there is no grid-wide barrier and CTAs of
// one launch need not be co-resident.  Flags carry a per-CTA launch counter that only grows, so
// they are never reset and a slow rank cannot confuse two launches.
//
// Algorithms
//   one-shot : every rank stores its packed chunk into slot [rank] of every peer's inbox, one
//              barrier, every rank sums the N local slots in rank order.  (N-1)*S bytes out per GPU,
//              one NVLink traversal of latency.  The inbox is double-buffered by launch parity.
//   two-shot : pack into the local staging buffer, barrier, rank r pulls sub-chunk r from all
//              peers and sums in rank order, stores the average into every peer's staging buffer,
//              barrier, every rank consumes its (now averaged) local buffer.  2*(N-1)/N*S bytes.
//   NVLS     : as two-shot, but the pull is one multimem.ld_reduce (the switch adds the N copies)
//              and the push one multimem.st on the multicast address of the staging buffer.
// With mode == 0 the two-shot / NVLS kernels stop after the second barrier: the averaged gradient is then
// complete in every rank's staging area, in the group's padded vector layout, for a later kernel to consume.
// Every rank applies the same arithmetic to the same reduced values, so replicas stay bit-identical.
//
// Every wait is bounded: after `timeout_ns` the CTA records (code, peer, expected, observed, cta) in
// the host-visible status block, skips the rest of its work and returns normally.
#include "api.h"

namespace {

constexpr int kUnroll = 4;      // float4 slots a thread keeps in flight in the streaming loops

struct Smem {
    int failed;
    float red[32];
};

// Checked build: thread 0 of every CTA stamps the end of each phase of the most recent launch
// (pack, first barrier, reduce, second barrier, consume of the FIRST piece, then the end of the last piece),
// nanoseconds since the CTA started.
#ifdef MGW_CHECKED
__device__ unsigned long long g_mgw_phase_ns[MGW_MAX_CTAS][6];
#define MGW_PHASE_BEGIN() const uint64_t phase_t0 = mgw_globaltimer_ns()
#define MGW_PHASE_END(i)                                                                    \
    do {                                                                                    \
        __syncthreads();                                                                    \
        if (threadIdx.x == 0) g_mgw_phase_ns[blockIdx.x][(i)] = mgw_globaltimer_ns() - phase_t0; \
    } while (0)
#else
#define MGW_PHASE_BEGIN() do {} while (0)
#define MGW_PHASE_END(i) do {} while (0)
#endif

__device__ __forceinline__ uint32_t* flag_slot(uint32_t* base, int phase, int cta, int src) {
    return base + ((size_t)(phase * MGW_MAX_CTAS + cta) * MGW_MAX_RANKS + src);
}

// CTA-to-CTA barrier across ranks.  Threads 0..world-1 each signal one peer and wait for that peer.
__device__ __forceinline__ bool rank_barrier(const MgwAllreduceArgs& a, int phase, uint32_t e, Smem* sm) {
    __syncthreads();                                   // this CTA's earlier stores are issued
    const int t = threadIdx.x;
    if (t < a.world) {
        __threadfence_system();
        mgw_st_release_sys(flag_slot(a.flags[t], phase, blockIdx.x, a.rank), e);
        uint32_t seen = 0;
        if (!mgw_wait_flag(flag_slot(a.flags[a.rank], phase, blockIdx.x, t), e, a.timeout_ns, &seen)) {
            mgw_report(a.status, MGW_STATUS_TIMEOUT, t, (int)e, (int)seen);
            sm->failed = 1;
        }
    }
    __syncthreads();
    return sm->failed == 0;
}

__device__ __forceinline__ float4 add4(float4 a, float4 b) {
    return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}

__device__ __forceinline__ float4 scale4(float4 a, float s) {
    return make_float4(a.x * s, a.y * s, a.z * s, a.w * s);
}

__device__ __forceinline__ float4 multimem_ld_reduce(const float4* mc) {
    float4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
    return v;
}

__device__ __forceinline__ void multimem_st(float4* mc, float4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
                 ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// W > 0: world size known at compile time (loops unroll); W == 0: read it from the arguments.
//
// Slot mapping of the streaming loops: per iteration a CTA covers blockDim.x * U consecutive slots,
// warp w of it the 32 * U slots starting at w * 32 * U, and a lane the U slots `lane + 32 k` of
// those, so every warp request is one contiguous 512-byte line group and the U slots of a thread
// lie within 1.5 KB of one another (the span that must fall inside one tensor for the table-free path).
template <int W, int ALGO>
__global__ void __launch_bounds__(512, 1) mgw_allreduce_kernel(const MgwAllreduceArgs a) {
    constexpr int WW = W > 0 ? W : MGW_MAX_RANKS;
    constexpr int U = kUnroll;                                  // pack / consume: one operand stream per slot
    constexpr int UR = (W == 1 || W == 2) ? 4 : (W == 4 ? 2 : 1);   // reduce: W peer loads per slot, keep ~8 in flight
    __shared__ Smem sm;
    const int world = W > 0 ? W : a.world;
    const int tid = threadIdx.x, nthr = blockDim.x, b = blockIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    if (tid == 0) sm.failed = 0;
    const uint32_t e = a.epoch[b] + 1u;
    const MgwGroup& g = a.group;
    const float inv = a.grad_scale / (float)world;

    // chunk of this CTA, a multiple of `world` slots so that sub-chunks are equal
    int per = (g.n_vec + gridDim.x - 1) / gridDim.x;
    per = (per + world - 1) / world * world;
    const int c0 = min(g.n_vec, b * per);
    const int c1 = min(g.n_vec, c0 + per);
    // two-shot / NVLS: number of pieces the chunk is processed in (same on every rank: it depends on the group's size
    // and the grid only); each piece uses one value of the CTA's launch counter
    const int pieces = ALGO == MGW_ALGO_ONESHOT ? 1 : max(1, min(a.max_pieces, per / max(a.piece_slots, 1)));
    float sumsq = 0.f;
    MGW_PHASE_BEGIN();
    // checked build: the chunk must lie inside the region the host sized; otherwise this CTA does nothing
    bool ok = MGW_CHECK(c1 <= (ALGO == MGW_ALGO_ONESHOT ? a.inbox_stride : a.stage_slots), MGW_BOUNDS_STAGE, c1,
                        ALGO == MGW_ALGO_ONESHOT ? a.inbox_stride : a.stage_slots, 0);

    if (!ok) {
        // fall through to the epoch update
    } else if (ALGO == MGW_ALGO_ONESHOT) {
        const size_t row = (size_t)a.inbox_stride;
        const size_t parity_base = (size_t)(e & 1u) * world * row;
        MgwCursor cl = mgw_cursor();
        for (int v0 = c0 + warp * 32 * U + lane; v0 < c1; v0 += nthr * U) {
            float4 x[U];
            mgw_load_grad_batch<U>(g, v0, 32, c1, cl, 1.f, x);
#pragma unroll
            for (int i = 0; i < WW; ++i) {
                if (i < world) {
                    int q = a.rank + 1 + i;
                    if (q >= world) q -= world;
                    float4* inbox = reinterpret_cast<float4*>(a.stage[q]) + parity_base + (size_t)a.rank * row;
#pragma unroll
                    for (int k = 0; k < U; ++k)
                        if (v0 + k * 32 < c1) mgw_st_peer(inbox + v0 + k * 32, x[k]);
                }
            }
        }
        ok = rank_barrier(a, 0, e, &sm);
        if (ok) {
            const float4* mine = reinterpret_cast<const float4*>(a.stage[a.rank]) + parity_base;
            MgwCursor cc = mgw_cursor();
            for (int v0 = c0 + warp * 32 * UR + lane; v0 < c1; v0 += nthr * UR) {
                float4 x[UR][WW];
#pragma unroll
                for (int k = 0; k < UR; ++k)
#pragma unroll
                    for (int s = 0; s < WW; ++s)
                        if (s < world && v0 + k * 32 < c1) x[k][s] = mgw_ld_peer(mine + (size_t)s * row + v0 + k * 32);
                float4 acc[UR];
#pragma unroll
                for (int k = 0; k < UR; ++k) {
                    acc[k] = x[k][0];
#pragma unroll
                    for (int s = 1; s < WW; ++s)
                        if (s < world) acc[k] = add4(acc[k], x[k][s]);
                    acc[k] = scale4(acc[k], inv);
                }
                mgw_consume_batch<UR>(g, v0, 32, c1, cc, acc, a.mode, a.hyper, a.first_step, sumsq);
            }
        }
    } else {
        // The chunk is cut into `pieces` consecutive pieces that go through pack / barrier / reduce / barrier /
        // consume one after another, each with its own flag value.  CTAs drift apart within a few pieces, so while
        // some wait on NVLink in the reduce phase others stream HBM in pack or consume, and with two CTAs per SM
        // a CTA that waits at a barrier leaves the SM to its neighbour.
        float4* local = reinterpret_cast<float4*>(a.stage[a.rank]);
        int plen = (per + pieces - 1) / pieces;
        plen = (plen + world - 1) / world * world;
        MgwCursor cur = mgw_cursor();          // one table cursor serves the pack and the consume loops of a piece
        for (int piece = 0; piece < pieces && ok; ++piece) {
            const uint32_t ep = e + (uint32_t)piece;
            const int p0 = min(c1, c0 + piece * plen);
            const int p1 = min(c1, p0 + plen);
            // skip_pack: copy-engine transfers queued ahead of this kernel already put the gradients into `local`
            // (same padded layout; the pad lanes of a tensor's last slot are never consumed)
            for (int v0 = p0 + warp * 32 * U + lane; v0 < p1 && !a.skip_pack; v0 += nthr * U) {
                float4 x[U];
                mgw_load_grad_batch<U>(g, v0, 32, p1, cur, 1.f, x);
#pragma unroll
                for (int k = 0; k < U; ++k)
                    if (v0 + k * 32 < p1) mgw_st_peer(local + v0 + k * 32, x[k]);
            }
            if (piece == 0) MGW_PHASE_END(0);
            ok = rank_barrier(a, 0, ep, &sm);
            if (piece == 0) MGW_PHASE_END(1);
            if (!ok) break;
            const int sub = plen / world;
            const int s0 = min(p1, p0 + a.rank * sub);
            const int s1 = min(p1, s0 + sub);
            if (ALGO == MGW_ALGO_NVLS) {
                float4* mc = reinterpret_cast<float4*>(a.mc_stage);
                for (int v0 = s0 + warp * 32 * U + lane; v0 < s1; v0 += nthr * U) {
                    float4 x[U];
#pragma unroll
                    for (int k = 0; k < U; ++k)
                        if (v0 + k * 32 < s1) x[k] = multimem_ld_reduce(mc + v0 + k * 32);
#pragma unroll
                    for (int k = 0; k < U; ++k)
                        if (v0 + k * 32 < s1) multimem_st(mc + v0 + k * 32, scale4(x[k], inv));
                }
            } else {
                for (int v0 = s0 + warp * 32 * UR + lane; v0 < s1; v0 += nthr * UR) {
                    float4 x[UR][WW];
#pragma unroll
                    for (int k = 0; k < UR; ++k)
#pragma unroll
                        for (int q = 0; q < WW; ++q)
                            if (q < world && v0 + k * 32 < s1)
                                x[k][q] = mgw_ld_peer(reinterpret_cast<const float4*>(a.stage[q]) + v0 + k * 32);
#pragma unroll
                    for (int k = 0; k < UR; ++k) {
                        float4 acc = x[k][0];
#pragma unroll
                        for (int q = 1; q < WW; ++q)
                            if (q < world) acc = add4(acc, x[k][q]);
                        x[k][0] = scale4(acc, inv);
                    }
#pragma unroll
                    for (int i = 0; i < WW; ++i) {
                        if (i < world) {
                            int q = a.rank + 1 + i;
                            if (q >= world) q -= world;
#pragma unroll
                            for (int k = 0; k < UR; ++k)
                                if (v0 + k * 32 < s1) mgw_st_peer(reinterpret_cast<float4*>(a.stage[q]) + v0 + k * 32, x[k][0]);
                        }
                    }
                }
            }
            if (piece == 0) MGW_PHASE_END(2);
            ok = rank_barrier(a, 1, ep, &sm);
            if (piece == 0) MGW_PHASE_END(3);
            if (!ok) break;
            // mode 0: the averaged gradient stays in the staging area and whoever launched the kernel reads it there
            // (the deferred update: one full-width SGD kernel after backward instead of an update inside every group)
            for (int v0 = p0 + warp * 32 * U + lane; v0 < p1 && a.mode != 0; v0 += nthr * U) {
                float4 x[U];
#pragma unroll
                for (int k = 0; k < U; ++k)
                    if (v0 + k * 32 < p1) x[k] = mgw_ld_peer(local + v0 + k * 32);
                mgw_consume_batch<U>(g, v0, 32, p1, cur, x, a.mode, a.hyper, a.first_step, sumsq);
            }
            if (piece == 0) MGW_PHASE_END(4);
        }
        MGW_PHASE_END(5);
    }

    if (a.mode & MGW_MODE_SUMSQ) {
        const float r = mgw_block_sum(ok ? sumsq : 0.f, sm.red);
        if (tid == 0) a.sumsq_partials[b] = r;
    }
    __syncthreads();
    if (tid == 0) a.epoch[b] = e + (uint32_t)(pieces - 1);      // advance even after a timeout: the launch counter stays in step
}

template <int ALGO>
cudaError_t launch_world(const MgwAllreduceArgs& a, cudaStream_t s) {
    dim3 grid(a.n_ctas), block(a.n_threads);
    switch (a.world) {
        case 1: mgw_allreduce_kernel<1, ALGO><<<grid, block, 0, s>>>(a); break;
        case 2: mgw_allreduce_kernel<2, ALGO><<<grid, block, 0, s>>>(a); break;
        case 4: mgw_allreduce_kernel<4, ALGO><<<grid, block, 0, s>>>(a); break;
        case 8: mgw_allreduce_kernel<8, ALGO><<<grid, block, 0, s>>>(a); break;
        default: mgw_allreduce_kernel<0, ALGO><<<grid, block, 0, s>>>(a); break;
    }
    return cudaGetLastError();
}

}  // namespace

MGW_DEFINE_BOUNDS_READER(mgw_bounds_allreduce)

// Checked build: per-CTA phase stamps of the most recent two-shot / NVLS launch, out[cta * 6 + phase] in ns
// (phases: pack, barrier, reduce, barrier, consume; slot 5 unused).  Zeros in the normal build.
extern "C" int mgw_phase_times(unsigned long long* out, int n_ctas) {
    if (out == nullptr || n_ctas < 1 || n_ctas > MGW_MAX_CTAS) return MGW_ERR_ARG;
#ifdef MGW_CHECKED
    MGW_CUDA_CHECK(cudaDeviceSynchronize());
    MGW_CUDA_CHECK(cudaMemcpyFromSymbol(out, g_mgw_phase_ns, sizeof(unsigned long long) * 6 * n_ctas));
#else
    for (int i = 0; i < 6 * n_ctas; ++i) out[i] = 0ull;
#endif
    return MGW_OK;
}

extern "C" size_t mgw_flag_block_bytes(void) {
    return sizeof(uint32_t) * 2 * MGW_MAX_CTAS * MGW_MAX_RANKS;
}

extern "C" size_t mgw_stage_bytes(int algo, int n_vec, int world) {
    const size_t one = (size_t)n_vec * sizeof(float4);
    return algo == MGW_ALGO_ONESHOT ? one * 2 * (size_t)world : one;
}

extern "C" int mgw_allreduce_group(const MgwAllreduceArgs* args, void* stream) {
    if (args == nullptr) return MGW_ERR_ARG;
    const MgwAllreduceArgs& a = *args;
    if (a.world < 1 || a.world > MGW_MAX_RANKS || a.rank < 0 || a.rank >= a.world) return MGW_ERR_ARG;
    if (a.n_ctas < 1 || a.n_ctas > MGW_MAX_CTAS) return MGW_ERR_ARG;
    if (a.n_threads < 32 || a.n_threads > 512 || (a.n_threads & 31) || a.n_threads < a.world) return MGW_ERR_ARG;
    if (a.group.n_vec < 0 || a.epoch == nullptr) return MGW_ERR_ARG;
    if ((a.mode & MGW_MODE_SUMSQ) && a.sumsq_partials == nullptr) return MGW_ERR_ARG;
    if ((a.mode & MGW_MODE_UPDATE) && a.hyper == nullptr) return MGW_ERR_ARG;
    if (a.algo == MGW_ALGO_NVLS && a.mc_stage == nullptr) return MGW_ERR_ARG;
    if (a.algo == MGW_ALGO_ONESHOT && a.inbox_stride < a.group.n_vec) return MGW_ERR_TOO_LARGE;
    if (a.algo != MGW_ALGO_ONESHOT && a.stage_slots < a.group.n_vec) return MGW_ERR_TOO_LARGE;
    if (a.algo != MGW_ALGO_ONESHOT && (a.max_pieces < 1 || a.piece_slots < 1)) return MGW_ERR_ARG;
    if (a.skip_pack && a.algo == MGW_ALGO_ONESHOT) return MGW_ERR_ARG;
    if (!(a.grad_scale > 0.f)) return MGW_ERR_ARG;
    for (int r = 0; r < a.world; ++r)
        if (a.stage[r] == nullptr || a.flags[r] == nullptr) return MGW_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t err;
    switch (a.algo) {
        case MGW_ALGO_ONESHOT: err = launch_world<MGW_ALGO_ONESHOT>(a, s); break;
        case MGW_ALGO_TWOSHOT: err = launch_world<MGW_ALGO_TWOSHOT>(a, s); break;
        case MGW_ALGO_NVLS: err = launch_world<MGW_ALGO_NVLS>(a, s); break;
        default: return MGW_ERR_ARG;
    }
    MGW_CUDA_CHECK(err);
    return MGW_OK;
}
