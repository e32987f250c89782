// Space-to-depth rearrangement of a 3-channel channels-last image batch, the input side of computing the
// ImageNet stem convolution (7x7, stride 2, padding 3, 3 input channels) as a 4x4 / stride 1 convolution over
// 12 channels: out[n, j, i, p*6 + q*3 + c] = x[n, 2j + p - 4, 2i + q - 4, c] (zero outside the image).
// For fixed (n, j, i, p) the six values (q, c) are contiguous in the source, so a thread moves 24 bytes
// with three 8-byte loads and stores.  One read of the image and one write of the rearranged copy; cuDNN's own
// handling of a 3-channel NHWC input costs a padding kernel, a layout conversion and legacy kernels instead.
#include "api.h"

namespace {

__global__ void __launch_bounds__(256)
s2d_stem_kernel(const float* __restrict__ x, float* __restrict__ out, int N, int H, int W, int OH, int OW) {
    const long long total = (long long)N * OH * OW * 2;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int p = (int)(idx & 1);
        long long t = idx >> 1;
        const int i = (int)(t % OW);
        t /= OW;
        const int j = (int)(t % OH);
        const long long n = t / OH;
        const int h = 2 * j + p - 4, w = 2 * i - 4;
        float2 a = make_float2(0.f, 0.f), b = a, c = a;
        if (h >= 0 && h < H && w >= 0 && w < W) {          // W is even and w is even, so w + 1 is inside too
            const float2* src = reinterpret_cast<const float2*>(x + ((n * H + h) * W + w) * 3);
            a = src[0]; b = src[1]; c = src[2];
        }
        float2* dst = reinterpret_cast<float2*>(out + ((n * OH + j) * OW + i) * 12 + p * 6);
        dst[0] = a; dst[1] = b; dst[2] = c;
    }
}

}  // namespace

// x: [N, H, W, 3] floats (channels-last image batch, H and W even); out: [N, H/2 + 3, W/2 + 3, 12] floats.
extern "C" int mgw_s2d_stem_input(const float* x, float* out, int N, int H, int W, void* stream) {
    if (x == nullptr || out == nullptr || N <= 0 || H <= 0 || W <= 0 || (H & 1) || (W & 1)) return MGW_ERR_ARG;
    const int OH = H / 2 + 3, OW = W / 2 + 3;
    const long long total = (long long)N * OH * OW * 2;
    const int grid = (int)((total + 255) / 256 < 148LL * 32 ? (total + 255) / 256 : 148LL * 32);
    s2d_stem_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(x, out, N, H, W, OH, OW);
    MGW_CUDA_CHECK(cudaGetLastError());
    return MGW_OK;
}
