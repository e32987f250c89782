// Recurrent matrix product of an LSTM time step for small batches:
//
//     P[s][b][r] = sum over k in K-range s of  X[b][k] * W[r][k]        b < B <= 64,  r < R,  s < KS
//
// X is the previous hidden state h_{t-1} [B, H] (forward: W = W_hh [4H, H]) or the gate gradients dG_t
// [B, 4H] (backward: W = W_hh^T [H, 4H]); the sums over the K-ranges are added up, in order, by the cell kernel
// that consumes P (lstm_cell.cu), so nothing here needs atomics and the result is deterministic.
//
// With B = 20 this is a matrix-vector product in disguise: every weight is used once per step and the step is
// bound by how fast the 36 MB of W_hh (H = 1500) come out of L2, not by arithmetic.  A library GEMM tiles for
// arithmetic intensity that is not there; this kernel is laid out for the stream instead:
//   * a CTA owns 64 rows of W and one K-range of 384 columns: 96 KB of weights, read exactly once, as 16-byte
//     loads that go straight into tensor-core fragments (no shared-memory staging of W);
//   * 8 warps = 4 row tiles x 2 halves of the K-range; every warp keeps 8 independent 16-byte loads in flight;
//   * the X slice of the K-range (at most 64 x 384 floats) is staged once in shared memory, padded so that the
//     fragment loads are conflict free;
//   * TF32 tensor-core MMAs (m16n8k8, fp32 accumulate, operands rounded to nearest).  The sixteen k of a chunk
//     are assigned to the two MMAs of the chunk in the order the 16-byte loads deliver them; A and B use the same
//     assignment, so no shuffle is needed.
// The warp-level mma.sync form is used on purpose: with N = B <= 64 and no operand reuse there is nothing a
// 128-row tcgen05 tile with TMEM accumulators could amortise.
#include "api.h"

namespace {

constexpr int kRowsPerCta = 64;
constexpr int kRange = 384;                  // K columns per CTA (multiple of 16)
constexpr int kThreads = 256;
constexpr int kXStride = kRange + 16;        // floats; (stride mod 32) == 16 keeps the float4 fragment loads conflict free

__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ void mma_tf32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT = number of 8-wide batch tiles (B <= 8 * NT)
template <int NT>
__global__ void __launch_bounds__(kThreads)
lstm_rec_gemm_kernel(const float* __restrict__ X, const float* __restrict__ W, float* __restrict__ P, int B, int R, int K) {
    extern __shared__ float xs[];                          // [8 * NT][kXStride]; later reused for the K-half reduction
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int wr = warp & 3, wk = warp >> 2;              // row tile (16 rows) and half of the K-range
    const int r0 = blockIdx.x * kRowsPerCta + wr * 16;
    const int kbeg = blockIdx.y * kRange;
    const int klen = min(kRange, K - kbeg);               // > 0 by construction of the grid; multiple of 4

    // stage the X slice: rows b >= B and columns beyond the range are zero
    for (int i = tid; i < 8 * NT * (kRange / 4); i += kThreads) {
        const int b = i / (kRange / 4), c4 = (i - b * (kRange / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b < B && c4 < klen) v = *reinterpret_cast<const float4*>(X + (size_t)b * K + kbeg + c4);
        *reinterpret_cast<float4*>(xs + b * kXStride + c4) = v;
    }
    __syncthreads();

    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    // rows beyond R read row R-1 again (valid memory); their results are never stored
    const float* w_lo = W + (size_t)min(r0 + g, R - 1) * K + kbeg;
    const float* w_hi = W + (size_t)min(r0 + g + 8, R - 1) * K + kbeg;
    const int c_first = wk * (kRange / 2), c_last = min(klen, c_first + kRange / 2);
    constexpr int U = 4;                                   // chunks of 16 columns in flight
    for (int c = c_first; c < c_last; c += 16 * U) {
        float4 a_lo[U], a_hi[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int col = c + 16 * u + 4 * t;
            if (col < c_last) {
                a_lo[u] = __ldg(reinterpret_cast<const float4*>(w_lo + col));
                a_hi[u] = __ldg(reinterpret_cast<const float4*>(w_hi + col));
            } else {
                a_lo[u] = a_hi[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int col = c + 16 * u + 4 * t;            // columns beyond c_last hold zeros in xs as well (or A is zero)
            const uint32_t l0 = to_tf32(a_lo[u].x), l1 = to_tf32(a_lo[u].y), l2 = to_tf32(a_lo[u].z), l3 = to_tf32(a_lo[u].w);
            const uint32_t h0 = to_tf32(a_hi[u].x), h1 = to_tf32(a_hi[u].y), h2 = to_tf32(a_hi[u].z), h3 = to_tf32(a_hi[u].w);
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const float4 xv = *reinterpret_cast<const float4*>(xs + (8 * n + g) * kXStride + min(col, kRange - 4));
                mma_tf32(acc[n], l0, h0, l1, h1, to_tf32(xv.x), to_tf32(xv.y));
                mma_tf32(acc[n], l2, h2, l3, h3, to_tf32(xv.z), to_tf32(xv.w));
            }
        }
    }

    // add the two K-halves (warps wk = 1 hand their sums to wk = 0 through shared memory), then store
    __syncthreads();                                       // everybody is done reading xs
    float* red = xs;                                       // [4 row tiles][32 lanes][NT * 4]
    if (wk == 1) {
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) red[(wr * 32 + lane) * (NT * 4) + n * 4 + i] = acc[n][i];
    }
    __syncthreads();
    if (wk == 0) {
        float* out = P + (size_t)blockIdx.y * B * R;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float v = acc[n][i] + red[(wr * 32 + lane) * (NT * 4) + n * 4 + i];
                const int r = r0 + g + ((i & 2) ? 8 : 0);
                const int b = 8 * n + 2 * t + (i & 1);
                if (r < R && b < B) out[(size_t)b * R + r] = v;
            }
        }
    }
}

}  // namespace

extern "C" {

// Number of K-ranges (= partial products) for an inner dimension of K.
int mgw_lstm_rec_splits(int K) { return K > 0 ? (K + kRange - 1) / kRange : 0; }

// 1 when the kernel handles the problem (fp32, 16-byte aligned rows, batch up to 64).
int mgw_lstm_rec_supported(const void* X, const void* W, int B, int R, int K) {
    if (B < 1 || B > 64 || R < 1 || K < 4 || (K & 3)) return 0;
    if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return 0;
    return 1;
}

// P [splits][B][R] (splits = mgw_lstm_rec_splits(K)) receives the partial products of X [B, K] and W [R, K]^T.
int mgw_lstm_rec_gemm(const float* X, const float* W, float* P, int B, int R, int K, void* stream) {
    if (!mgw_lstm_rec_supported(X, W, B, R, K) || P == nullptr) return MGW_ERR_ARG;
    const dim3 grid((R + kRowsPerCta - 1) / kRowsPerCta, mgw_lstm_rec_splits(K)), block(kThreads);
    const int nt = (B + 7) / 8;
    const size_t smem = sizeof(float) * 8 * nt * kXStride;       // >= the reduction area (4 * 32 * nt * 4 floats)
    cudaStream_t s = (cudaStream_t)stream;
#define MGW_REC_CASE(N)                                                                                          \
    case N: {                                                                                                    \
        static bool configured = false;                                                                          \
        if (!configured && smem > 48 * 1024) {                                                                   \
            MGW_CUDA_CHECK(cudaFuncSetAttribute(lstm_rec_gemm_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
            configured = true;                                                                                   \
        }                                                                                                        \
        lstm_rec_gemm_kernel<N><<<grid, block, smem, s>>>(X, W, P, B, R, K);                                     \
        break;                                                                                                   \
    }
    switch (nt) {
        MGW_REC_CASE(1) MGW_REC_CASE(2) MGW_REC_CASE(3) MGW_REC_CASE(4) MGW_REC_CASE(5) MGW_REC_CASE(6) MGW_REC_CASE(7) MGW_REC_CASE(8)
        default: return MGW_ERR_ARG;
    }
#undef MGW_REC_CASE
    MGW_CUDA_CHECK(cudaGetLastError());
    return MGW_OK;
}

}  // extern "C"
