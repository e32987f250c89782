// Weight-gradient GEMM for large fully-connected / LSTM layers on Blackwell tensor cores:
//
//     dW[M, N] = sum_k  dY[k, m] * X[k, n]        (M = out features, N = in features, K = batch rows)
//
// with dY stored [K, M] and X stored [K, N] row-major, i.e. BOTH operands are "MN-major": K is the
// slow dimension of both.  K is small (64 rows per GPU for the VGG classifier, 700 for the PTB
// LSTM), so the kernel is bound by its output, not by math: a 128x128 fp32 tile is 64 KB of result
// for 2*128*128*K flops.  That is why the epilogue does the optimizer work in place: instead of
// writing dW and having an all-reduce and an SGD kernel read it back, the tile leaves tensor memory
// once and is applied to the weights and momentum directly (optionally also stored as a gradient).
//
// Data-parallel use: every rank first all-gathers the K-rows of dY and X of all ranks into local
// buffers (mgw_allgather_rows below: peer loads over NVLink, bounded flag waits).  That moves
// W*B*(M+N) floats instead of all-reducing M*N of them (7.4 MB instead of 411 MB for the
// 25088 -> 4096 VGG layer on 8 GPUs), and every rank then runs this same GEMM over K = W*B rows in
// the same order, so replicas stay bit-identical.
//
// Two kernels share the pieces below.  The default is the persistent one further down (a CTA per SM walks over the
// tiles; 299 us for the 4096 x 25088 layer with the SGD epilogue, 0.85 of the measured copy bandwidth, against 375 us
// for the one-tile form and 99 us against the library's 91 us when only the gradient is stored).  The one-tile form:
// structure of one CTA (320 threads, one 128x128 output tile, three CTAs per SM):
//   warp 0   : TMA producer.  Per K-block of 32 rows: four 2-D tiled bulk-tensor loads of
//              [32 rows x 32 floats] for each operand (128-byte swizzle with 32-byte atoms), completing
//              on an mbarrier.
//   warp 1   : allocates 128 tensor-memory columns, then one lane issues tcgen05.mma kind::tf32
//              (M=128, N=128, K=8 per instruction, both operands MN-major from shared memory) and
//              commits each stage back to the producer and the finished tile to the epilogue.
//   warps 2-9: epilogue, two warps per tensor-memory lane quarter.  tcgen05.ld (32 lanes x 32 columns)
//              -> swizzled staging in the (by then idle) operand stages -> 256-byte row segments of
//              W / momentum / gradient in global memory, optimizer applied in registers.
// Every mbarrier wait is bounded; on expiry the CTA records an error, lets its outstanding bulk
// copies land (bounded as well), frees its tensor memory and returns.
#include <cuda.h>
#include <cstdlib>
#include "api.h"

namespace {

constexpr int BM = 128, BN = 128, BK = 32;
constexpr int kStages = 2;
constexpr int kAtomFloats = 32;                       // swizzle atom = 32 floats (128 bytes) along M or N
constexpr int kRegionBytes = BK * 128;                // one [BK x 32 floats] box
constexpr int kAStageBytes = (BM / kAtomFloats) * kRegionBytes;   // 16 KB
constexpr int kBStageBytes = (BN / kAtomFloats) * kRegionBytes;   // 16 KB
constexpr int kStageBytes = kAStageBytes + kBStageBytes;
constexpr int kEpiWarps = 8;                          // two per tensor-memory lane quarter, 64 columns each
constexpr int kThreadsPerCta = 64 + 32 * kEpiWarps;   // producer warp + MMA warp + epilogue warps
constexpr int kEpiWarpFloats = 32 * 64;               // one warp stages 32 rows x 64 columns (8 KB)
static_assert(kEpiWarps * kEpiWarpFloats * 4 <= kStages * kStageBytes, "epilogue staging reuses the operand stages");
constexpr int kSmemBytes = 1024 + kStages * kStageBytes + 256;
constexpr int kTmemCols = 128;
constexpr uint32_t kWaitSpins = 1u << 22;

#define WG_MODE_STORE 1      // write dW * scale to `grad_out`
#define WG_MODE_SGD 2        // apply dW * scale to (weight, momentum) with the hyper-parameters of `pg`
#define WG_MODE_SCATTER 4    // reduce-scatter epilogue: store the tile into its OWNER rank's staging slot (peer stores)

struct Params {
    float* weight;
    float* mom;
    float* grad_out;
    const MgwHyper* hyper;
    int* status;
    int M, N, K;
    int mode, pg, first_step;
    float scale;
    // WG_MODE_SCATTER: tile t (row-major over the tile grid) belongs to rank t % world; rank r's copy of it goes to
    // scatter[owner] + (r * tiles_per_owner + t / world) * BM * BN, a full 128 x 128 slot (rows beyond M / N hold zeros)
    float* const* scatter;
    int rank, world, tiles_per_owner;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// Bounded parity wait.  Returns false when the phase did not complete within the spin limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < kWaitSpins; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if (spin > 1024) __nanosleep(32);
    }
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

// Shared-memory matrix descriptor for an MN-major 32-bit operand.  The only shared-memory layout the
// tensor cores accept for that case is the 128-byte swizzle with 32-byte granularity: an atom is
// 32 floats along M/N by 4 rows of K (512 bytes), 32-byte chunks of a row are permuted by the row
// index mod 4.  `lbo` = bytes between consecutive atoms along M/N, `sbo` = bytes between consecutive
// 4-row atoms along K.  The bulk-tensor loads use the matching swizzle mode.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;                 // descriptor version for this architecture
    d |= 1ull << 61;                 // 128-byte swizzle, 32-byte base
    return d;
}

// Instruction descriptor: D = F32, A = B = TF32, both operands MN-major, M = 128, N = 128.
__device__ __forceinline__ uint32_t make_instr_desc() {
    return (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void report(int* status, int code) {
    if (status) atomicCAS_system(status, 0, code);      // the word may live in pinned host memory
}

__global__ void __launch_bounds__(kThreadsPerCta, 3)
wgrad_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stages = smem;                                           // kStages x (A | B), 1024-byte aligned
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
    uint64_t* full = bars;                     // [kStages]
    uint64_t* empty = bars + kStages;          // [kStages]
    uint64_t* acc_ready = bars + 2 * kStages;  // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 1);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int num_kb = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_ready, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int issued = 0;
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % kStages;
                const uint32_t ph = (kb / kStages) & 1;
                if (!mbar_wait(&empty[s], ph ^ 1)) { report(p.status, 11); *failed = 1; break; }
                if (*failed) break;
                uint8_t* a_dst = stages + s * kStageBytes;
                uint8_t* b_dst = a_dst + kAStageBytes;
                mbar_expect_tx(&full[s], kStageBytes);
#pragma unroll
                for (int j = 0; j < BM / kAtomFloats; ++j) tma_load_2d(a_dst + j * kRegionBytes, &map_a, m0 + j * kAtomFloats, kb * BK, &full[s]);
#pragma unroll
                for (int j = 0; j < BN / kAtomFloats; ++j) tma_load_2d(b_dst + j * kRegionBytes, &map_b, n0 + j * kAtomFloats, kb * BK, &full[s]);
                issued = kb + 1;
            }
            if (*failed) {
                // let copies that were already issued land before the CTA gives up its shared memory
                for (int kb = max(0, issued - kStages); kb < issued; ++kb) (void)mbar_wait(&full[kb % kStages], (kb / kStages) & 1);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = make_instr_desc();
            bool ok = true;
            for (int kb = 0; kb < num_kb && ok; ++kb) {
                const int s = kb % kStages;
                const uint32_t ph = (kb / kStages) & 1;
                if (!mbar_wait(&full[s], ph) || *failed) { report(p.status, 12); *failed = 1; ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_u32(stages + s * kStageBytes);
                const uint32_t b_addr = a_addr + kAStageBytes;
#pragma unroll
                for (int kk = 0; kk < BK / 8; ++kk) {
                    const uint64_t adesc = make_smem_desc(a_addr + kk * 1024, kRegionBytes, 512);
                    const uint64_t bdesc = make_smem_desc(b_addr + kk * 1024, kRegionBytes, 512);
                    umma_tf32(tmem_base, adesc, bdesc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(&empty[s]);          // the stage may be refilled once these MMAs have read it
            }
            umma_commit(acc_ready);              // arrives when every MMA issued above has completed
        }
    } else {
        // ---------------- epilogue (warps 2..9) ----------------
        // Warp w may read tensor-memory lanes 32*(w%4)..+31, i.e. 32 rows of the tile; two warps share a lane
        // quarter and split the 128 columns.  Once the accumulator is complete every MMA has finished reading
        // the operand stages, so each warp reuses 8 KB of them to turn its rows (one thread = one row out of
        // tensor memory) into 256-byte row segments (16 threads = one row segment) for global memory.
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;
        float4* wsm = reinterpret_cast<float4*>(stages) + (size_t)(warp - 2) * (kEpiWarpFloats / 4);
        bool ok = mbar_wait(acc_ready, 0);
        if (!ok) { report(p.status, 13); *failed = 1; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok && !*failed) {
            MgwHyper h;
            if (p.mode & WG_MODE_SGD) h = p.hyper[p.pg];
#pragma unroll
            for (int cb = 0; cb < 2; ++cb) {
                float v[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(half * 64 + cb * 32), v);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const int chunk = cb * 8 + c;
                    wsm[lane * 16 + (chunk ^ (lane & 7))] =
                        make_float4(v[4 * c] * p.scale, v[4 * c + 1] * p.scale, v[4 * c + 2] * p.scale, v[4 * c + 3] * p.scale);
                }
            }
            __syncwarp();
            const int ch = lane & 15;
            if (p.mode & WG_MODE_SCATTER) {
                // The tile leaves tensor memory once and goes straight into the reduction: 256-byte row segments into the
                // owner's slot for this rank, over NVLink when the owner is a peer (ordinary stores; the finishing
                // kernel's barrier publishes them).
                const int t = blockIdx.y * gridDim.x + blockIdx.x;
                const int owner = t % p.world;
                float* slot = p.scatter[owner] + ((size_t)p.rank * p.tiles_per_owner + (size_t)(t / p.world)) * (BM * BN);
#pragma unroll 4
                for (int i = 0; i < 16; ++i) {
                    const int rr = 2 * i + (lane >> 4);
                    const float4 g = wsm[rr * 16 + (ch ^ (rr & 7))];
                    mgw_st_peer(reinterpret_cast<float4*>(slot + (size_t)(q * 32 + rr) * BN + half * 64 + 4 * ch), g);
                }
            }
            const int n = n0 + half * 64 + 4 * ch;
            const bool use_m = (p.mode & WG_MODE_SGD) && p.mom != nullptr && h.momentum != 0.f;
#pragma unroll 4
            for (int i = 0; i < 16; ++i) {
                const int rr = 2 * i + (lane >> 4);
                const int m = m0 + q * 32 + rr;
                if (m < p.M && n < p.N) {
                    float4 g = wsm[rr * 16 + (ch ^ (rr & 7))];
                    const size_t off = (size_t)m * p.N + n;
                    if (p.mode & WG_MODE_STORE) *reinterpret_cast<float4*>(p.grad_out + off) = g;
                    if (p.mode & WG_MODE_SGD) {
                        float4 w = *reinterpret_cast<float4*>(p.weight + off);
                        float4 mo = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (use_m && !p.first_step) mo = *reinterpret_cast<float4*>(p.mom + off);
                        mgw_sgd_scalar(g.x, w.x, use_m ? &mo.x : nullptr, h, p.first_step);
                        mgw_sgd_scalar(g.y, w.y, use_m ? &mo.y : nullptr, h, p.first_step);
                        mgw_sgd_scalar(g.z, w.z, use_m ? &mo.z : nullptr, h, p.first_step);
                        mgw_sgd_scalar(g.w, w.w, use_m ? &mo.w : nullptr, h, p.first_step);
                        *reinterpret_cast<float4*>(p.weight + off) = w;
                        if (use_m) *reinterpret_cast<float4*>(p.mom + off) = mo;
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }

    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ---- persistent form ----------------------------------------------------------------------------------
// CTAs that stay on their SM walk over the output tiles (tile = blockIdx.x, + gridDim.x, ...).  The three roles
// run as pipelines that are decoupled by mbarriers, so the bulk loads and MMAs of tile i+1 run while the epilogue
// warps still stream tile i through global memory:
//   warp 0 : TMA producer over a ring of kSt operand stages that is shared by consecutive tiles;
//   warp 1 : MMA issuer; accumulators alternate between two 128-column halves of 256 tensor-memory columns
//            (acc_empty / acc_full barriers per half);
//   warps 2.. : kEW epilogue warps, kEW / 4 per tensor-memory lane quarter.  A warp works through its share of the
//            tile's columns in blocks of 32: it copies the 32 x 32 block out of tensor memory, releases the
//            accumulator after its last block (the MMAs of the tile after next may start), transposes through
//            4 KB of its own shared memory and applies the block to 128-byte row segments of W / momentum /
//            gradient, four rows' loads in flight at a time.
// Two shapes are built: 16 epilogue warps + 4 stages with one CTA per SM, and 8 epilogue warps + 2 stages with two
// CTAs per SM (512 tensor-memory columns in total either way).
// Waits are bounded as in the one-tile kernel; after a failure every role leaves its loop, the producer
// lets its outstanding copies land, and the tensor memory is freed after the common barrier.
constexpr int kPEpiWarpBytes = 32 * 32 * 4;
constexpr int kPTmemCols = 256;
constexpr int persistent_smem_bytes(int epi_warps, int n_stages) { return 1024 + n_stages * kStageBytes + epi_warps * kPEpiWarpBytes + 256; }

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// W and momentum of four rows (rows r0 + 4 i + rsub) at column n: independent 16-byte loads, all in flight together
__device__ __forceinline__ void epi_load4(const Params& p, bool sgd, bool load_m, int m_first, int n, float4 (&w)[4], float4 (&mo)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m_first + 4 * i;
        w[i] = mo[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (sgd && m < p.M && n < p.N) {
            const size_t off = (size_t)m * p.N + n;
            w[i] = *reinterpret_cast<const float4*>(p.weight + off);
            if (load_m) mo[i] = *reinterpret_cast<const float4*>(p.mom + off);
        }
    }
}

__device__ __forceinline__ void epi_apply4(const Params& p, const MgwHyper& h, bool use_m, const float4* wsm, int ch, int rr_first, int m_first,
                                           int n, float4 (&w)[4], float4 (&mo)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int rr = rr_first + 4 * i, m = m_first + 4 * i;
        if (m >= p.M || n >= p.N) continue;
        float4 g = wsm[rr * 8 + (ch ^ (rr & 7))];
        const size_t off = (size_t)m * p.N + n;
        if (p.mode & WG_MODE_STORE) *reinterpret_cast<float4*>(p.grad_out + off) = g;
        if (p.mode & WG_MODE_SGD) {
            mgw_sgd_scalar(g.x, w[i].x, use_m ? &mo[i].x : nullptr, h, p.first_step);
            mgw_sgd_scalar(g.y, w[i].y, use_m ? &mo[i].y : nullptr, h, p.first_step);
            mgw_sgd_scalar(g.z, w[i].z, use_m ? &mo[i].z : nullptr, h, p.first_step);
            mgw_sgd_scalar(g.w, w[i].w, use_m ? &mo[i].w : nullptr, h, p.first_step);
            *reinterpret_cast<float4*>(p.weight + off) = w[i];
            if (use_m) *reinterpret_cast<float4*>(p.mom + off) = mo[i];
        }
    }
}

template <int kEW, int kSt, int kMinCtas>
__global__ void __launch_bounds__(64 + 32 * kEW, kMinCtas)
wgrad_gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
    static_assert(kEW % 4 == 0 && kEW >= 4 && kEW <= 16, "whole sets of four lane quarters");
    constexpr int kPasses = BN / 32 / (kEW / 4);                      // 32-column blocks per epilogue warp and tile
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stages = smem;                                           // kSt x (A | B), 1024-byte aligned
    uint8_t* epi = smem + kSt * kStageBytes;                          // kEW x 4 KB
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi + kEW * kPEpiWarpBytes);
    uint64_t* full = bars;                     // [kSt]
    uint64_t* empty = bars + kSt;              // [kSt]
    uint64_t* acc_full = bars + 2 * kSt;       // [2]
    uint64_t* acc_empty = bars + 2 * kSt + 2;  // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kSt + 4);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (p.K + BK - 1) / BK;
    const int tiles_x = (p.N + BN - 1) / BN, tiles_y = (p.M + BM - 1) / BM;
    const int num_tiles = tiles_x * tiles_y;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kSt; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], kEW);
        }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kPTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;                                  // k-blocks issued so far, over all tiles of this CTA
            for (int tile = blockIdx.x; tile < num_tiles && !*failed; tile += gridDim.x) {
                const int m0 = (tile / tiles_x) * BM, n0 = (tile % tiles_x) * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const uint32_t s = it % kSt, ph = (it / kSt) & 1;
                    if (!mbar_wait(&empty[s], ph ^ 1)) { report(p.status, 21); *failed = 1; }
                    if (*failed) break;
                    uint8_t* a_dst = stages + s * kStageBytes;
                    uint8_t* b_dst = a_dst + kAStageBytes;
                    mbar_expect_tx(&full[s], kStageBytes);
#pragma unroll
                    for (int j = 0; j < BM / kAtomFloats; ++j) tma_load_2d(a_dst + j * kRegionBytes, &map_a, m0 + j * kAtomFloats, kb * BK, &full[s]);
#pragma unroll
                    for (int j = 0; j < BN / kAtomFloats; ++j) tma_load_2d(b_dst + j * kRegionBytes, &map_b, n0 + j * kAtomFloats, kb * BK, &full[s]);
                }
            }
            if (*failed) {
                // let copies that were already issued land before the CTA gives up its shared memory
                for (uint32_t j = (it > (uint32_t)kSt ? it - kSt : 0u); j < it; ++j) (void)mbar_wait(&full[j % kSt], (j / kSt) & 1);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = make_instr_desc();
            uint32_t it = 0, tl = 0;                          // k-blocks consumed, tiles started
            for (int tile = blockIdx.x; tile < num_tiles && !*failed; tile += gridDim.x, ++tl) {
                const uint32_t a = tl & 1, aph = (tl >> 1) & 1;
                if (!mbar_wait(&acc_empty[a], aph ^ 1)) { report(p.status, 22); *failed = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + a * (uint32_t)BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const uint32_t s = it % kSt, ph = (it / kSt) & 1;
                    if (!mbar_wait(&full[s], ph)) { report(p.status, 23); *failed = 1; }
                    if (*failed) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(stages + s * kStageBytes);
                    const uint32_t b_addr = a_addr + kAStageBytes;
#pragma unroll
                    for (int kk = 0; kk < BK / 8; ++kk) {
                        const uint64_t adesc = make_smem_desc(a_addr + kk * 1024, kRegionBytes, 512);
                        const uint64_t bdesc = make_smem_desc(b_addr + kk * 1024, kRegionBytes, 512);
                        umma_tf32(tmem_d, adesc, bdesc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[s]);          // the stage may be refilled once these MMAs have read it
                }
                if (*failed) break;
                umma_commit(&acc_full[a]);           // arrives when every MMA of this tile has completed
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int q = warp & 3;                              // tensor-memory lane quarter this warp may read
        const int cq = (warp - 2) >> 2;                      // which share of the tile's columns
        float4* wsm = reinterpret_cast<float4*>(epi + (size_t)(warp - 2) * kPEpiWarpBytes);
        MgwHyper h;
        const bool sgd = (p.mode & WG_MODE_SGD) != 0;
        if (sgd) h = p.hyper[p.pg];
        const bool use_m = sgd && p.mom != nullptr && h.momentum != 0.f;
        const bool load_m = use_m && !p.first_step;
        const int ch = lane & 7, rsub = lane >> 3;
        uint32_t tl = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tl) {
            const uint32_t a = tl & 1, aph = (tl >> 1) & 1;
            const int m0 = (tile / tiles_x) * BM + q * 32;
#pragma unroll
            for (int cb = 0; cb < kPasses; ++cb) {
                const int col0 = (cq * kPasses + cb) * 32;              // column block within the tile
                const int n = (tile % tiles_x) * BN + col0 + 4 * ch;
                float4 w0[4], mo0[4], w1[4], mo1[4];
                if (cb == 0) {
                    if (*failed || !mbar_wait(&acc_full[a], aph)) {
                        if (!*failed) { report(p.status, 24); *failed = 1; }
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                }
                float v[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + a * (uint32_t)BN + (uint32_t)col0, v);
                if (cb == kPasses - 1) asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();                                // also: every lane is done reading the previous block's staging
                if (cb == kPasses - 1 && lane == 0) mbar_arrive(&acc_empty[a]);
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    wsm[lane * 8 + (c ^ (lane & 7))] = make_float4(v[4 * c] * p.scale, v[4 * c + 1] * p.scale, v[4 * c + 2] * p.scale, v[4 * c + 3] * p.scale);
                __syncwarp();
                if (p.mode & WG_MODE_SCATTER) {
                    const int owner = tile % p.world;
                    float* slot = p.scatter[owner] + ((size_t)p.rank * p.tiles_per_owner + (size_t)(tile / p.world)) * (BM * BN);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rr = 4 * i + rsub;
                        mgw_st_peer(reinterpret_cast<float4*>(slot + (size_t)(q * 32 + rr) * BN + col0 + 4 * ch), wsm[rr * 8 + (ch ^ (rr & 7))]);
                    }
                }
                if (p.mode & (WG_MODE_STORE | WG_MODE_SGD)) {
                    // Four rows (eight 16-byte loads per thread) in flight at a time.  Issuing these loads earlier, before
                    // the wait for the accumulator, measured 410 instead of 299 us on the 4096 x 25088 layer.
                    epi_load4(p, sgd, load_m, m0 + rsub, n, w0, mo0);
                    epi_apply4(p, h, use_m, wsm, ch, rsub, m0 + rsub, n, w0, mo0);
                    epi_load4(p, sgd, load_m, m0 + 16 + rsub, n, w1, mo1);
                    epi_apply4(p, h, use_m, wsm, ch, 16 + rsub, m0 + 16 + rsub, n, w1, mo1);
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }

    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kPTmemCols) : "memory");
    }
}

// ---- all-gather of K-row blocks over NVLink -----------------------------------------------------------
// Every rank contributes `block_floats` floats (its block lives at offset rank*block_floats of its own
// symmetric buffer); afterwards every rank holds all W blocks in rank order.  Pull design with two
// bounded barriers per CTA: "my block is in place" before the copy, "I am done reading" after it, so a
// rank may overwrite its block for the next step as soon as its own kernel has finished.
__device__ __forceinline__ bool gather_barrier(uint32_t* const* flags, int phase, int rank, int world, uint32_t e, int* status,
                                               unsigned long long timeout_ns, int* failed) {
    __syncthreads();
    if (threadIdx.x < world) {
        __threadfence_system();
        const size_t slot = ((size_t)phase * MGW_MAX_CTAS + blockIdx.x) * MGW_MAX_RANKS;
        mgw_st_release_sys(flags[threadIdx.x] + slot + rank, e);
        uint32_t seen = 0;
        if (!mgw_wait_flag(flags[rank] + slot + threadIdx.x, e, timeout_ns, &seen)) {
            mgw_report(status, MGW_STATUS_TIMEOUT, threadIdx.x, (int)e, (int)seen);
            *failed = 1;
        }
    }
    __syncthreads();
    return *failed == 0;
}

__global__ void __launch_bounds__(512)
allgather_rows_kernel(float* const* bufs, uint32_t* const* flags, uint32_t* epoch, int* status, int rank, int world,
                      long long block_floats, unsigned long long timeout_ns) {
    __shared__ int failed;
    const int b = blockIdx.x;
    const uint32_t e = epoch[b] + 1u;
    if (threadIdx.x == 0) failed = 0;
    if (gather_barrier(flags, 0, rank, world, e, status, timeout_ns, &failed)) {
        const long long nvec = block_floats / 4;
        const long long per = (nvec + gridDim.x - 1) / gridDim.x;
        const long long v0 = (long long)b * per, v1 = min(nvec, v0 + per);
        for (int i = 1; i < world; ++i) {
            int q = rank + i;
            if (q >= world) q -= world;
            const float4* src = reinterpret_cast<const float4*>(bufs[q] + (size_t)q * block_floats);
            float4* dst = reinterpret_cast<float4*>(bufs[rank] + (size_t)q * block_floats);
            for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) dst[v] = mgw_ld_peer(src + v);
        }
        (void)gather_barrier(flags, 1, rank, world, e, status, timeout_ns, &failed);
    }
    __syncthreads();
    if (threadIdx.x == 0) epoch[b] = e;
}

// Second half of the reduce-scatter weight gradient: runs on every rank behind its own scatter GEMM.  After a barrier
// ("every rank's tiles are in the owners' slots") rank r adds up, in rank order, the `world` slots of each tile it owns
// and stores the sum into EVERY rank's gradient tensor (symmetric memory, ordinary peer stores); a second barrier says
// "every gradient tensor is complete".  Sums are formed once, by one rank, and broadcast: replicas get identical bits.
__global__ void __launch_bounds__(512)
wgrad_reduce_finish_kernel(float* const* stage, float* const* grads, uint32_t* const* flags, uint32_t* epoch, int* status, int rank,
                           int world, int M, int N, int tiles_per_owner, unsigned long long timeout_ns) {
    __shared__ int failed;
    const int b = blockIdx.x;
    const uint32_t e = epoch[b] + 1u;
    if (threadIdx.x == 0) failed = 0;
    if (gather_barrier(flags, 0, rank, world, e, status, timeout_ns, &failed)) {
        const int tiles_x = (N + BN - 1) / BN, tiles_y = (M + BM - 1) / BM;
        const int tiles = tiles_x * tiles_y;
        const int owned = (tiles - rank + world - 1) / world;            // tiles t with t % world == rank
        const float4* mine = reinterpret_cast<const float4*>(stage[rank]);
        constexpr int kTileVec = BM * BN / 4;
        for (int ti = b; ti < owned; ti += gridDim.x) {
            const int t = ti * world + rank;
            const int m0 = (t / tiles_x) * BM, n0 = (t % tiles_x) * BN;
            for (int v = threadIdx.x; v < kTileVec; v += blockDim.x) {
                const int row = v / (BN / 4), col = (v - row * (BN / 4)) * 4;
                const int m = m0 + row, n = n0 + col;
                if (m >= M || n >= N) continue;
                float4 acc = mgw_ld_peer(mine + (size_t)ti * kTileVec + v);
                for (int s = 1; s < world; ++s) {
                    const float4 x = mgw_ld_peer(mine + ((size_t)s * tiles_per_owner + ti) * kTileVec + v);
                    acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
                }
                const size_t off = (size_t)m * N + n;
                for (int i = 0; i < world; ++i) {
                    int q = rank + i;
                    if (q >= world) q -= world;
                    mgw_st_peer(reinterpret_cast<float4*>(grads[q] + off), acc);
                }
            }
        }
        (void)gather_barrier(flags, 1, rank, world, e, status, timeout_ns, &failed);
    }
    __syncthreads();
    if (threadIdx.x == 0) epoch[b] = e;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// [K rows, inner floats] row-major operand -> boxes of [BK rows x 32 floats], 128-byte swizzle with 32-byte atoms.
bool make_map(CUtensorMap* map, const float* base, int K, int inner) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return false;
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)K};
    cuuint64_t strides[1] = {(cuuint64_t)inner * sizeof(float)};
    cuuint32_t box[2] = {(cuuint32_t)kAtomFloats, (cuuint32_t)BK};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}


// Which form runs: 2 = persistent, two CTAs of 8 epilogue warps per SM; 1 = persistent, one CTA of 16 epilogue warps per SM;
// 0 = one tile per CTA.  MGWFBP_WGRAD_PERSISTENT in the environment, or mgw_wgrad_set_persistent() at run time.
int g_persistent = -1;
constexpr int kDefaultForm = 1;

int persistent_sms(int* sms) {
    constexpr int kMaxDevices = 64;
    static int cached[kMaxDevices];
    int dev = 0;
    MGW_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return MGW_ERR_ARG;
    if (cached[dev] == 0) {
        int n = 0;
        MGW_CUDA_CHECK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
        cached[dev] = n > 0 ? n : 1;
    }
    *sms = cached[dev];
    return MGW_OK;
}

template <int kEW, int kSt, int kMinCtas>
int launch_persistent(const CUtensorMap& map_a, const CUtensorMap& map_b, const Params& p, long long n_tiles, cudaStream_t stream) {
    constexpr int smem = persistent_smem_bytes(kEW, kSt);
    static bool configured = false;
    if (!configured) {
        MGW_CUDA_CHECK(cudaFuncSetAttribute(wgrad_gemm_persistent_kernel<kEW, kSt, kMinCtas>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured = true;
    }
    int sms = 0;
    const int rc = persistent_sms(&sms);
    if (rc != MGW_OK) return rc;
    const long long slots = (long long)sms * kMinCtas;
    wgrad_gemm_persistent_kernel<kEW, kSt, kMinCtas><<<(int)(n_tiles < slots ? n_tiles : slots), 64 + 32 * kEW, smem, stream>>>(map_a, map_b, p);
    return MGW_OK;
}

int launch_gemm(const CUtensorMap& map_a, const CUtensorMap& map_b, const Params& p, cudaStream_t stream) {
    if (g_persistent < 0) {
        const char* e = getenv("MGWFBP_WGRAD_PERSISTENT");
        g_persistent = (e == nullptr || e[0] < '0' || e[0] > '2') ? kDefaultForm : e[0] - '0';
    }
    const dim3 tiles((p.N + BN - 1) / BN, (p.M + BM - 1) / BM);
    const long long n_tiles = (long long)tiles.x * tiles.y;
    int rc = MGW_OK;
    if (g_persistent == 2) {
        rc = launch_persistent<8, 2, 2>(map_a, map_b, p, n_tiles, stream);
    } else if (g_persistent == 1) {
        rc = launch_persistent<16, 4, 1>(map_a, map_b, p, n_tiles, stream);
    } else {
        static bool configured = false;
        if (!configured) {
            MGW_CUDA_CHECK(cudaFuncSetAttribute(wgrad_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
            configured = true;
        }
        wgrad_gemm_kernel<<<tiles, kThreadsPerCta, kSmemBytes, stream>>>(map_a, map_b, p);
    }
    if (rc != MGW_OK) return rc;
    MGW_CUDA_CHECK(cudaGetLastError());
    return MGW_OK;
}

}  // namespace

extern "C" {

// 2 / 1: persistent kernel (two CTAs of 8 epilogue warps / one CTA of 16 per SM), 0: one tile per CTA, negative: read
// MGWFBP_WGRAD_PERSISTENT again at the next launch.
void mgw_wgrad_set_persistent(int form) { g_persistent = form < 0 ? -1 : (form > 2 ? 2 : form); }

// 1 when the shapes meet the kernel's alignment rules (16-byte aligned bases, M and N multiples of 4).
int mgw_wgrad_gemm_supported(const void* dy, const void* x, int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if ((M & 3) || (N & 3)) return 0;
    if ((reinterpret_cast<uintptr_t>(dy) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return 0;
    return 1;
}

// dy: [K, M], x: [K, N] row-major fp32.  mode bit 1: grad_out[M, N] = scale * dy^T x;
// mode bit 2: momentum-SGD on (weight, mom) with hyper[pg].  status: one device-visible int (0 = ok).
int mgw_wgrad_gemm(const float* dy, const float* x, int M, int N, int K, float scale, int mode, float* grad_out, float* weight,
                   float* mom, const MgwHyper* hyper, int pg, int first_step, int* status, void* stream) {
    if (!mgw_wgrad_gemm_supported(dy, x, M, N, K)) return MGW_ERR_ARG;
    if ((mode & WG_MODE_STORE) && grad_out == nullptr) return MGW_ERR_ARG;
    if ((mode & WG_MODE_SGD) && (weight == nullptr || hyper == nullptr)) return MGW_ERR_ARG;
    if ((mode & (WG_MODE_STORE | WG_MODE_SGD)) == 0) return MGW_ERR_ARG;
    CUtensorMap map_a, map_b;
    if (!make_map(&map_a, dy, K, M) || !make_map(&map_b, x, K, N)) {
        mgw_set_last_error(cudaErrorUnknown, "cuTensorMapEncodeTiled", __FILE__, __LINE__);
        return MGW_ERR_CUDA;
    }
    Params p;
    p.weight = weight; p.mom = mom; p.grad_out = grad_out; p.hyper = hyper; p.status = status;
    p.M = M; p.N = N; p.K = K; p.mode = mode; p.pg = pg; p.first_step = first_step; p.scale = scale;
    p.scatter = nullptr; p.rank = 0; p.world = 1; p.tiles_per_owner = 0;
    return launch_gemm(map_a, map_b, p, (cudaStream_t)stream);
}

// Floats of staging every rank must provide for the reduce-scatter form of an [M, N] weight gradient on `world` ranks:
// `world` source rows of ceil(tiles / world) full 128 x 128 slots.
size_t mgw_wgrad_scatter_stage_floats(int M, int N, int world) {
    if (M <= 0 || N <= 0 || world < 1) return 0;
    const size_t tiles = (size_t)((N + BN - 1) / BN) * (size_t)((M + BM - 1) / BM);
    return (size_t)world * ((tiles + world - 1) / world) * (size_t)(BM * BN);
}

// First half of the reduce-scatter weight gradient: scale * dy^T x, each 128 x 128 tile stored into the staging area of
// the rank that owns it (stage_dev: device array of every rank's staging base, peers included).  Nothing is written
// locally.  Follow it on the same stream with mgw_wgrad_reduce_finish.
int mgw_wgrad_gemm_scatter(const float* dy, const float* x, int M, int N, int K, float scale, float* const* stage_dev, int rank,
                           int world, int* status, void* stream) {
    if (!mgw_wgrad_gemm_supported(dy, x, M, N, K) || stage_dev == nullptr) return MGW_ERR_ARG;
    if (world < 1 || world > MGW_MAX_RANKS || rank < 0 || rank >= world) return MGW_ERR_ARG;
    CUtensorMap map_a, map_b;
    if (!make_map(&map_a, dy, K, M) || !make_map(&map_b, x, K, N)) {
        mgw_set_last_error(cudaErrorUnknown, "cuTensorMapEncodeTiled", __FILE__, __LINE__);
        return MGW_ERR_CUDA;
    }
    Params p;
    p.weight = nullptr; p.mom = nullptr; p.grad_out = nullptr; p.hyper = nullptr; p.status = status;
    p.M = M; p.N = N; p.K = K; p.mode = WG_MODE_SCATTER; p.pg = 0; p.first_step = 0; p.scale = scale;
    const size_t tiles = (size_t)((N + BN - 1) / BN) * (size_t)((M + BM - 1) / BM);
    p.scatter = stage_dev; p.rank = rank; p.world = world; p.tiles_per_owner = (int)((tiles + world - 1) / world);
    return launch_gemm(map_a, map_b, p, (cudaStream_t)stream);
}

// Second half: owners add their slots up in rank order and store the sums into every rank's gradient tensor
// (grads_dev: device array of every rank's [M, N] gradient in symmetric memory).  flags / epoch as in mgw_allgather_rows,
// with rows of their own.  Both waits are bounded by timeout_ns.
int mgw_wgrad_reduce_finish(float* const* stage_dev, float* const* grads_dev, uint32_t* const* flags_dev, uint32_t* epoch, int* status,
                            int rank, int world, int M, int N, int n_ctas, unsigned long long timeout_ns, void* stream) {
    if (stage_dev == nullptr || grads_dev == nullptr || flags_dev == nullptr || epoch == nullptr) return MGW_ERR_ARG;
    if (world < 1 || world > MGW_MAX_RANKS || rank < 0 || rank >= world || n_ctas < 1 || n_ctas > MGW_MAX_CTAS) return MGW_ERR_ARG;
    if (M <= 0 || N <= 0 || (N & 3)) return MGW_ERR_ARG;
    const size_t tiles = (size_t)((N + BN - 1) / BN) * (size_t)((M + BM - 1) / BM);
    wgrad_reduce_finish_kernel<<<n_ctas, 512, 0, (cudaStream_t)stream>>>(stage_dev, grads_dev, flags_dev, epoch, status, rank, world, M, N,
                                                                       (int)((tiles + world - 1) / world), timeout_ns);
    MGW_CUDA_CHECK(cudaGetLastError());
    return MGW_OK;
}

// flags: every rank's flag block (same layout and size as mgw_flag_block_bytes()); epoch: local [MGW_MAX_CTAS] counters.
int mgw_allgather_rows(float* const* bufs_dev, uint32_t* const* flags_dev, uint32_t* epoch, int* status, int rank, int world,
                       long long block_floats, int n_ctas, unsigned long long timeout_ns, void* stream) {
    if (bufs_dev == nullptr || flags_dev == nullptr || epoch == nullptr) return MGW_ERR_ARG;
    if (world < 1 || world > MGW_MAX_RANKS || rank < 0 || rank >= world || n_ctas < 1 || n_ctas > MGW_MAX_CTAS) return MGW_ERR_ARG;
    if (block_floats <= 0 || (block_floats & 3)) return MGW_ERR_ARG;
    allgather_rows_kernel<<<n_ctas, 512, 0, (cudaStream_t)stream>>>(bufs_dev, flags_dev, epoch, status, rank, world, block_floats, timeout_ns);
    MGW_CUDA_CHECK(cudaGetLastError());
    return MGW_OK;
}

}  // extern "C"
