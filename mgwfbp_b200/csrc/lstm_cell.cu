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

}  // namespace

// gh: `gh_parts` (>= 1) partial recurrent products [B, 4H], `gh_stride` floats apart.
extern "C" int mgw_lstm_cell_fwd(const float* gx, const float* gh, const float* b_ih, const float* b_hh, const float* c_prev,
                                 float* h_out, float* c_out, float* act, int B, int H, int gh_parts, long long gh_stride, void* stream) {
    if (!gx || !gh || !c_prev || !h_out || !c_out || B <= 0 || H <= 0 || gh_parts < 1) return MGW_ERR_ARG;
    const int n = B * H;
    lstm_cell_fwd_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(gx, gh, b_ih, b_hh, c_prev, h_out, c_out, act, B, H,
                                                                           gh_parts, gh_stride);
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
    lstm_cell_bwd_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(dh, dc_in, act, c_prev, c_cur, dgates, dc_prev, B, H,
                                                                           dh_rec, dh_parts, dh_stride);
    MGW_CUDA_CHECK(cudaGetLastError());
    return MGW_OK;
}
