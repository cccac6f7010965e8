// Direct 2-D cross-correlation for the reference's single-channel conv2d (lib/autogradEngine/tensor.dart:765-833)
// and Conv2DLayer (lib/layertypes/conv2d.dart:60-75: every kernel of the layer over the same input matrix, plus a
// scalar bias per kernel).  With one input channel and k x k taps the contraction length is k*k (9, 25): far too
// short for the tensor cores, so these are streaming kernels: one thread per output (or input) element, taps read
// through the read-only cache, x fastest so that every warp touches contiguous rows.
//
// Layouts: in [n_img][H][W], w [n_k][kh][kw], out / dout [n_img][n_k][OH][OW], OH = H + 2 pad - kh + 1.
// 'same' padding is pad = (kh - 1) / 2 on every side (tensor.dart:773-776); padded positions contribute to neither
// gradient (the `continue` at tensor.dart:813-818).  All gradients accumulate (+=) like the reference's closure.
#include "common.cuh"

namespace {

constexpr int CV_THREADS = 256;
inline int cv_blocks(fml_ctx* ctx, long long n) {
  return (int)std::max<long long>(1, std::min<long long>((n + CV_THREADS - 1) / CV_THREADS, (long long)ctx->sm_count * 8));
}

__global__ void __launch_bounds__(CV_THREADS) conv2d_fwd_kernel(const float* __restrict__ in, const float* __restrict__ w,
                                                                const float* __restrict__ bias, float* __restrict__ out,
                                                                int n_img, int H, int W, int n_k, int kh, int kw, int pad, int OH,
                                                                int OW) {
  const long long total = (long long)n_img * n_k * OH * OW;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int x = (int)(i % OW);
    long long r = i / OW;
    const int y = (int)(r % OH);
    r /= OH;
    const int c = (int)(r % n_k);
    const int b = (int)(r / n_k);
    const float* img = in + (size_t)b * H * W;
    const float* wk = w + (size_t)c * kh * kw;
    float sum = 0.f;
    for (int ky = 0; ky < kh; ky++) {
      const int iy = y + ky - pad;
      if (iy < 0 || iy >= H) continue;
      for (int kx = 0; kx < kw; kx++) {
        const int ix = x + kx - pad;
        if (ix >= 0 && ix < W) sum = fmaf(__ldg(img + (size_t)iy * W + ix), __ldg(wk + ky * kw + kx), sum);
      }
    }
    out[i] = sum + (bias ? __ldg(bias + c) : 0.f);
  }
}

// din[b][iy][ix] += sum_c sum_k w[c][ky][kx] * dout[b][c][iy + pad - ky][ix + pad - kx]
__global__ void __launch_bounds__(CV_THREADS) conv2d_bwd_input_kernel(const float* __restrict__ w, const float* __restrict__ dout,
                                                                      float* din, int n_img, int H, int W, int n_k, int kh, int kw,
                                                                      int pad, int OH, int OW) {
  const long long total = (long long)n_img * H * W;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int ix = (int)(i % W);
    const long long r = i / W;
    const int iy = (int)(r % H);
    const int b = (int)(r / H);
    float sum = 0.f;
    for (int c = 0; c < n_k; c++) {
      const float* g = dout + ((size_t)b * n_k + c) * OH * OW;
      const float* wk = w + (size_t)c * kh * kw;
      for (int ky = 0; ky < kh; ky++) {
        const int y = iy + pad - ky;
        if (y < 0 || y >= OH) continue;
        for (int kx = 0; kx < kw; kx++) {
          const int x = ix + pad - kx;
          if (x >= 0 && x < OW) sum = fmaf(__ldg(wk + ky * kw + kx), __ldg(g + (size_t)y * OW + x), sum);
        }
      }
    }
    din[i] += sum;
  }
}

__device__ __forceinline__ float cv_block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  if (threadIdx.x < CV_THREADS / 32) t = red[threadIdx.x];
  if (threadIdx.x < 32) {
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  return t;  // valid in thread 0
}

// dw[c][ky][kx] += sum_b sum_yx in[b][y + ky - pad][x + kx - pad] * dout[b][c][y][x]; blockIdx.x = tap, blockIdx.y = slice
// of the (b, y, x) range; one atomic per block.  tap == n_k*kh*kw .. n_k*kh*kw + n_k - 1 are the bias gradients.
__global__ void __launch_bounds__(CV_THREADS) conv2d_bwd_weight_kernel(const float* __restrict__ in, const float* __restrict__ dout,
                                                                       float* dw, float* dbias, int n_img, int H, int W, int n_k,
                                                                       int kh, int kw, int pad, int OH, int OW) {
  __shared__ float red[CV_THREADS / 32];
  const int taps = n_k * kh * kw;
  const int tap = blockIdx.x;
  const bool is_bias = tap >= taps;
  const int c = is_bias ? tap - taps : tap / (kh * kw);
  const int ky = is_bias ? 0 : (tap / kw) % kh, kx = is_bias ? 0 : tap % kw;
  const long long per_img = (long long)OH * OW, total = (long long)n_img * per_img;
  float acc = 0.f;
  for (long long i = blockIdx.y * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.y * blockDim.x) {
    const int b = (int)(i / per_img);
    const long long r = i - (long long)b * per_img;
    const int y = (int)(r / OW), x = (int)(r - (long long)y * OW);
    const float g = __ldg(dout + ((size_t)b * n_k + c) * per_img + r);
    if (is_bias) {
      acc += g;
    } else {
      const int iy = y + ky - pad, ix = x + kx - pad;
      if (iy >= 0 && iy < H && ix >= 0 && ix < W) acc = fmaf(__ldg(in + ((size_t)b * H + iy) * W + ix), g, acc);
    }
  }
  const float t = cv_block_sum(acc, red);
  if (threadIdx.x == 0) atomicAdd(is_bias ? dbias + c : dw + tap, t);
}

}  // namespace

extern "C" {

int32_t fml_conv2d_fwd(fml_ctx* ctx, const float* in, const float* w, const float* bias, float* out, int32_t n_img, int32_t H,
                       int32_t W, int32_t n_k, int32_t kh, int32_t kw, int32_t pad) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, in && w && out && n_img > 0 && H > 0 && W > 0 && n_k > 0 && kh > 0 && kw > 0 && pad >= 0, "fml_conv2d_fwd: bad arguments");
  const int OH = H + 2 * pad - kh + 1, OW = W + 2 * pad - kw + 1;
  FML_REQUIRE(ctx, OH > 0 && OW > 0, "fml_conv2d_fwd: kernel larger than the padded input");
  conv2d_fwd_kernel<<<cv_blocks(ctx, (long long)n_img * n_k * OH * OW), CV_THREADS, 0, ctx->stream>>>(in, w, bias, out, n_img, H, W, n_k,
                                                                                                      kh, kw, pad, OH, OW);
  FML_LAUNCH_CHECK(ctx, "conv2d_fwd_kernel");
  return FML_OK;
}

int32_t fml_conv2d_bwd(fml_ctx* ctx, const float* in, const float* w, const float* dout, float* din, float* dw, float* dbias,
                       int32_t n_img, int32_t H, int32_t W, int32_t n_k, int32_t kh, int32_t kw, int32_t pad) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, in && w && dout && n_img > 0 && H > 0 && W > 0 && n_k > 0 && kh > 0 && kw > 0 && pad >= 0, "fml_conv2d_bwd: bad arguments");
  const int OH = H + 2 * pad - kh + 1, OW = W + 2 * pad - kw + 1;
  FML_REQUIRE(ctx, OH > 0 && OW > 0, "fml_conv2d_bwd: kernel larger than the padded input");
  if (din) {
    conv2d_bwd_input_kernel<<<cv_blocks(ctx, (long long)n_img * H * W), CV_THREADS, 0, ctx->stream>>>(w, dout, din, n_img, H, W, n_k, kh,
                                                                                                      kw, pad, OH, OW);
    FML_LAUNCH_CHECK(ctx, "conv2d_bwd_input_kernel");
  }
  if (dw || dbias) {
    // taps first, then (optionally) one pseudo-tap per kernel for its bias; skipped outputs are never launched
    const int taps = n_k * kh * kw;
    const int count = (dw ? taps : 0) + (dbias ? n_k : 0);
    const long long total = (long long)n_img * OH * OW;
    int slices = (int)std::max<long long>(1, std::min<long long>((total + CV_THREADS * 8 - 1) / (CV_THREADS * 8),
                                                                 ((long long)ctx->sm_count * 8 + count - 1) / count));
    slices = std::min(slices, 65535);
    if (dw && dbias) {
      conv2d_bwd_weight_kernel<<<dim3(count, slices), CV_THREADS, 0, ctx->stream>>>(in, dout, dw, dbias, n_img, H, W, n_k, kh, kw, pad, OH, OW);
    } else if (dw) {
      conv2d_bwd_weight_kernel<<<dim3(taps, slices), CV_THREADS, 0, ctx->stream>>>(in, dout, dw, nullptr, n_img, H, W, n_k, kh, kw, pad, OH, OW);
    } else {
      // bias only: shift the tap origin so that blockIdx.x = 0 is the first bias
      conv2d_bwd_weight_kernel<<<dim3(n_k, slices), CV_THREADS, 0, ctx->stream>>>(in, dout, nullptr, dbias, n_img, H, W, n_k, 0, 0, pad, OH, OW);
    }
    FML_LAUNCH_CHECK(ctx, "conv2d_bwd_weight_kernel");
  }
  return FML_OK;
}

}  // extern "C"
