// LSTM cell pointwise kernels (forward and backward).
//
// One LSTM time step is  gates = x_t W_ih^T + h_{t-1} W_hh^T + b_ih + b_hh  followed by
//   i = sigmoid(g_i)  f = sigmoid(g_f)  g = tanh(g_g)  o = sigmoid(g_o)
//   c_t = f * c_{t-1} + i * g        h_t = o * tanh(c_t)
// (gate order i, f, g, o as in torch.nn.LSTM).  The two matrix products stay library GEMMs; these
// kernels fuse everything after them: the sum of the two GEMM outputs, both biases, the four
// activations and the state update, in one pass, keeping the activated gates for the backward
// pass.  The backward kernel turns (dh_t, dc_t) into the gradient of the pre-activation gates and
// dc_{t-1}, again in one pass.  Layout: gates [B, 4H] row-major, states [B, H].
// The recurrent product may arrive as several partial sums over ranges of the inner dimension (the
// split-K output of lstm_rec.cu): `parts` arrays `stride` floats apart, added here in index order.
#include "api.h"

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

__global__ void __launch_bounds__(256)
lstm_cell_fwd_kernel(const float* __restrict__ gx, const float* __restrict__ gh, const float* __restrict__ b_ih,
                     const float* __restrict__ b_hh, const float* __restrict__ c_prev, float* __restrict__ h_out,
                     float* __restrict__ c_out, float* __restrict__ act, int B, int H, int parts, long long stride) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= B * H) return;
    const int b = idx / H, j = idx - b * H;
    const size_t row = (size_t)b * 4 * H;
    float g[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float r = gh[row + k * H + j];
        for (int p = 1; p < parts; ++p) r += gh[(size_t)p * stride + row + k * H + j];
        float v = gx[row + k * H + j] + r;
        if (b_ih) v += b_ih[k * H + j];
        if (b_hh) v += b_hh[k * H + j];
        g[k] = v;
    }
    const float i = sigmoidf_(g[0]), f = sigmoidf_(g[1]), gg = tanhf(g[2]), o = sigmoidf_(g[3]);
    const float c = fmaf(f, c_prev[idx], i * gg);
    c_out[idx] = c;
    h_out[idx] = o * tanhf(c);
    if (act) {
        act[row + 0 * H + j] = i;
        act[row + 1 * H + j] = f;
        act[row + 2 * H + j] = gg;
        act[row + 3 * H + j] = o;
    }
}

__global__ void __launch_bounds__(256)
lstm_cell_bwd_kernel(const float* __restrict__ dh, const float* __restrict__ dc_in, const float* __restrict__ act,
                     const float* __restrict__ c_prev, const float* __restrict__ c_cur, float* __restrict__ dgates,
                     float* __restrict__ dc_prev, int B, int H, const float* __restrict__ dh_rec, int parts, long long stride) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= B * H) return;
    const int b = idx / H, j = idx - b * H;
    const size_t row = (size_t)b * 4 * H;
    const float i = act[row + j], f = act[row + H + j], g = act[row + 2 * H + j], o = act[row + 3 * H + j];
    const float tc = tanhf(c_cur[idx]);
    float dhv = dh ? dh[idx] : 0.f;                           // gradient arriving from the layer above / the loss ...
    for (int p = 0; p < parts; ++p) dhv += dh_rec[(size_t)p * stride + idx];      // ... plus the one through h_t -> gates_{t+1}
    float dc = dhv * o * (1.f - tc * tc);
    if (dc_in) dc += dc_in[idx];
    dgates[row + j] = dc * g * i * (1.f - i);
    dgates[row + H + j] = dc * c_prev[idx] * f * (1.f - f);
    dgates[row + 2 * H + j] = dc * i * (1.f - g * g);
    dgates[row + 3 * H + j] = dhv * tc * o * (1.f - o);
    dc_prev[idx] = dc * f;
}

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }

// Four hidden units per thread (H % 4 == 0, 16-byte aligned rows): every access is one 16-byte transaction.
__global__ void __launch_bounds__(128)
lstm_cell_fwd_vec_kernel(const float* __restrict__ gx, const float* __restrict__ gh, const float* __restrict__ b_ih,
                         const float* __restrict__ b_hh, const float* __restrict__ c_prev, float* __restrict__ h_out,
                         float* __restrict__ c_out, float* __restrict__ act, int B, int H, int parts, long long stride) {
    const int q = blockIdx.x * blockDim.x + threadIdx.x;          // index of a group of four hidden units
    const int hq = H >> 2;
    if (q >= B * hq) return;
    const int b = q / hq, j = (q - b * hq) << 2;
    const size_t row = (size_t)b * 4 * H;
    float4 g[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float4 v = add4(ld4(gx + row + k * H + j), ld4(gh + row + k * H + j));
        for (int p = 1; p < parts; ++p) v = add4(v, ld4(gh + (size_t)p * stride + row + k * H + j));
        if (b_ih) v = add4(v, ld4(b_ih + k * H + j));
        if (b_hh) v = add4(v, ld4(b_hh + k * H + j));
        g[k] = v;
    }
    const float4 cp = ld4(c_prev + (size_t)b * H + j);
    float4 i4, f4, g4, o4, c4, h4;
#define MGW_CELL(X)                                                                   \
    i4.X = sigmoidf_(g[0].X); f4.X = sigmoidf_(g[1].X); g4.X = tanhf(g[2].X); o4.X = sigmoidf_(g[3].X); \
    c4.X = fmaf(f4.X, cp.X, i4.X * g4.X); h4.X = o4.X * tanhf(c4.X);
    MGW_CELL(x) MGW_CELL(y) MGW_CELL(z) MGW_CELL(w)
#undef MGW_CELL
    st4(c_out + (size_t)b * H + j, c4);
    st4(h_out + (size_t)b * H + j, h4);
    if (act) {
        st4(act + row + j, i4); st4(act + row + H + j, f4); st4(act + row + 2 * H + j, g4); st4(act + row + 3 * H + j, o4);
    }
}

__global__ void __launch_bounds__(128)
lstm_cell_bwd_vec_kernel(const float* __restrict__ dh, const float* __restrict__ dc_in, const float* __restrict__ act,
                         const float* __restrict__ c_prev, const float* __restrict__ c_cur, float* __restrict__ dgates,
                         float* __restrict__ dc_prev, int B, int H, const float* __restrict__ dh_rec, int parts, long long stride) {
    const int q = blockIdx.x * blockDim.x + threadIdx.x;
    const int hq = H >> 2;
    if (q >= B * hq) return;
    const int b = q / hq, j = (q - b * hq) << 2;
    const size_t row = (size_t)b * 4 * H, s = (size_t)b * H + j;
    const float4 i4 = ld4(act + row + j), f4 = ld4(act + row + H + j), g4 = ld4(act + row + 2 * H + j), o4 = ld4(act + row + 3 * H + j);
    const float4 cc = ld4(c_cur + s), cp = ld4(c_prev + s);
    float4 dhv = dh ? ld4(dh + s) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < parts; ++p) dhv = add4(dhv, ld4(dh_rec + (size_t)p * stride + s));
    const float4 dci = dc_in ? ld4(dc_in + s) : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 di, df, dg, dox, dcp;
#define MGW_CELL(X)                                                                   \
    {                                                                                 \
        const float tc = tanhf(cc.X);                                                 \
        const float dc = dhv.X * o4.X * (1.f - tc * tc) + dci.X;                      \
        di.X = dc * g4.X * i4.X * (1.f - i4.X);                                       \
        df.X = dc * cp.X * f4.X * (1.f - f4.X);                                       \
        dg.X = dc * i4.X * (1.f - g4.X * g4.X);                                       \
        dox.X = dhv.X * tc * o4.X * (1.f - o4.X);                                     \
        dcp.X = dc * f4.X;                                                            \
    }
    MGW_CELL(x) MGW_CELL(y) MGW_CELL(z) MGW_CELL(w)
#undef MGW_CELL
    st4(dgates + row + j, di); st4(dgates + row + H + j, df); st4(dgates + row + 2 * H + j, dg); st4(dgates + row + 3 * H + j, dox);
    st4(dc_prev + s, dcp);
}

inline bool aligned16(const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

// gh: `gh_parts` (>= 1) partial recurrent products [B, 4H], `gh_stride` floats apart.
extern "C" int mgw_lstm_cell_fwd(const float* gx, const float* gh, const float* b_ih, const float* b_hh, const float* c_prev,
                                 float* h_out, float* c_out, float* act, int B, int H, int gh_parts, long long gh_stride, void* stream) {
    if (!gx || !gh || !c_prev || !h_out || !c_out || B <= 0 || H <= 0 || gh_parts < 1) return MGW_ERR_ARG;
    const int n = B * H;
    if ((H & 3) == 0 && (gh_stride & 3) == 0 && aligned16(gx) && aligned16(gh) && aligned16(b_ih) && aligned16(b_hh) &&
        aligned16(c_prev) && aligned16(h_out) && aligned16(c_out) && aligned16(act)) {
        lstm_cell_fwd_vec_kernel<<<(n / 4 + 127) / 128, 128, 0, (cudaStream_t)stream>>>(gx, gh, b_ih, b_hh, c_prev, h_out, c_out, act,
                                                                                       B, H, gh_parts, gh_stride);
    } else {
        lstm_cell_fwd_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(gx, gh, b_ih, b_hh, c_prev, h_out, c_out, act, B, H,
                                                                               gh_parts, gh_stride);
    }
    MGW_CUDA_CHECK(cudaGetLastError());
    return MGW_OK;
}

// dh (may be null): gradient of h_t from outside the recurrence; dh_rec (may be null when dh_parts == 0): `dh_parts`
// partial products dG_{t+1} W_hh [B, H], `dh_stride` floats apart.  Their sum is the gradient of h_t.
extern "C" int mgw_lstm_cell_bwd(const float* dh, const float* dc_in, const float* act, const float* c_prev, const float* c_cur,
                                 float* dgates, float* dc_prev, int B, int H, const float* dh_rec, int dh_parts, long long dh_stride,
                                 void* stream) {
    if (!act || !c_prev || !c_cur || !dgates || !dc_prev || B <= 0 || H <= 0 || dh_parts < 0 || (dh_parts > 0 && !dh_rec))
        return MGW_ERR_ARG;
    const int n = B * H;
    if ((H & 3) == 0 && (dh_stride & 3) == 0 && aligned16(dh) && aligned16(dc_in) && aligned16(act) && aligned16(c_prev) &&
        aligned16(c_cur) && aligned16(dgates) && aligned16(dc_prev) && aligned16(dh_rec)) {
        lstm_cell_bwd_vec_kernel<<<(n / 4 + 127) / 128, 128, 0, (cudaStream_t)stream>>>(dh, dc_in, act, c_prev, c_cur, dgates, dc_prev,
                                                                                       B, H, dh_rec, dh_parts, dh_stride);
    } else {
        lstm_cell_bwd_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(dh, dc_in, act, c_prev, c_cur, dgates, dc_prev, B, H,
                                                                               dh_rec, dh_parts, dh_stride);
    }
    MGW_CUDA_CHECK(cudaGetLastError());
    return MGW_OK;
}
