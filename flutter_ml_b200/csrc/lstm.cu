// LSTM layer over a batch of sequences, built from the contraction kernels plus two fused
// gate kernels.  The input projection of ALL timesteps is one large GEMM (bias folded into its
// epilogue); each timestep then adds the recurrent product h_{t-1}.Wh^T into its slice with a
// beta = 1 epilogue and runs one kernel that applies the four gate nonlinearities and the cell
// update.  BPTT mirrors it: one gate-gradient kernel and one small GEMM per step, then the
// weight gradients of all timesteps as two large GEMMs.
//
// Reference: LSTMLayer.forward lib/layertypes/lstmLayer.dart:112-150.  Gate order f,i,c~,o
// (:64); weight columns [h_{t-1} | x_t] (:119).
#include <algorithm>

#include "common.cuh"

namespace {

__device__ __forceinline__ float sigf(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float tanh_ref(float x) {
  float e2x = expf(2.f * x);
  return isinf(e2x) ? 1.f : (e2x - 1.f) / (e2x + 1.f);
}

// pre [B][4H] -> activated gates (in a separate buffer), c_t, h_t
__global__ void lstm_gates_fwd_kernel(const float* __restrict__ pre, const float* __restrict__ c_prev,
                                      float* __restrict__ gates, float* __restrict__ c_out, float* __restrict__ h_out,
                                      int B, int H) {
  const int n = B * H;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += gridDim.x * blockDim.x) {
    const int b = idx / H, r = idx - b * H;
    const float* p = pre + (long long)b * 4 * H;
    const float f = sigf(p[r]), i = sigf(p[H + r]), g = tanh_ref(p[2 * H + r]), o = sigf(p[3 * H + r]);
    const float c = f * c_prev[idx] + i * g;
    float* gt = gates + (long long)b * 4 * H;
    gt[r] = f; gt[H + r] = i; gt[2 * H + r] = g; gt[3 * H + r] = o;
    c_out[idx] = c;
    h_out[idx] = o * tanh_ref(c);
  }
}

// dh, dc (in/out: becomes dc_{t-1}), saved gates and cells -> gradient of the pre-activations
__global__ void lstm_gates_bwd_kernel(const float* __restrict__ dh, float* dc, const float* __restrict__ gates,
                                      const float* __restrict__ c_prev, const float* __restrict__ c_cur,
                                      float* __restrict__ dpre, int B, int H) {
  const int n = B * H;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += gridDim.x * blockDim.x) {
    const int b = idx / H, r = idx - b * H;
    const float* gt = gates + (long long)b * 4 * H;
    const float f = gt[r], i = gt[H + r], g = gt[2 * H + r], o = gt[3 * H + r];
    const float tc = tanh_ref(c_cur[idx]);
    const float dhv = dh[idx];
    const float d_o = dhv * tc;
    const float dct = dc[idx] + dhv * o * (1.f - tc * tc);
    float* dp = dpre + (long long)b * 4 * H;
    dp[r] = dct * c_prev[idx] * (f * (1.f - f));
    dp[H + r] = dct * g * (i * (1.f - i));
    dp[2 * H + r] = dct * i * (1.f - g * g);
    dp[3 * H + r] = d_o * (o * (1.f - o));
    dc[idx] = dct * f;
  }
}

inline int blocks_for(fml_ctx* ctx, long long n) {
  return (int)std::max<long long>(1, std::min<long long>((n + 255) / 256, (long long)ctx->sm_count * 4));
}

fml_gemm_desc gemm_defaults() {
  fml_gemm_desc g = {};
  g.alpha = 1.f;
  g.batch1 = g.batch2 = 1;
  g.precision = -1;
  return g;
}

}  // namespace

extern "C" {

int32_t fml_lstm_fwd(fml_ctx* ctx, const fml_lstm_desc* d) {
  FML_REQUIRE(ctx, d && d->W && d->b && d->x && d->gates && d->cells && d->hs && d->xproj, "fml_lstm_fwd: NULL buffer");
  FML_REQUIRE(ctx, d->T > 0 && d->B > 0 && d->I > 0 && d->H > 0, "fml_lstm_fwd: bad sizes");
  const int T = d->T, B = d->B, I = d->I, H = d->H, Z = H + I;
  const long long bh = (long long)B * H, b4h = (long long)B * 4 * H;
  FML_CUDA(ctx, cudaMemsetAsync(d->cells, 0, bh * 4, ctx->stream));
  FML_CUDA(ctx, cudaMemsetAsync(d->hs, 0, bh * 4, ctx->stream));
  // xproj[T*B][4H] = x . Wx^T + b   (Wx = columns H.. of W)
  fml_gemm_desc g = gemm_defaults();
  g.M = T * B; g.N = 4 * H; g.K = I;
  g.A = d->x; g.lda = I;
  g.B = d->W + H; g.ldb = Z; g.transB = 1;
  g.C = d->xproj; g.ldc = 4 * H;
  g.bias = d->b;
  int32_t rc = fml_gemm(ctx, &g);
  if (rc) return rc;
  for (int t = 0; t < T; t++) {
    float* pre = d->xproj + t * b4h;
    if (t > 0) {
      fml_gemm_desc r = gemm_defaults();
      r.M = B; r.N = 4 * H; r.K = H;
      r.A = d->hs + t * bh; r.lda = H;
      r.B = d->W; r.ldb = Z; r.transB = 1;
      r.C = pre; r.ldc = 4 * H; r.beta = 1.f;
      if ((rc = fml_gemm(ctx, &r))) return rc;
    }
    lstm_gates_fwd_kernel<<<blocks_for(ctx, bh), 256, 0, ctx->stream>>>(pre, d->cells + t * bh, d->gates + t * b4h,
                                                                        d->cells + (t + 1) * bh, d->hs + (t + 1) * bh, B, H);
  }
  FML_LAUNCH_CHECK(ctx, "lstm_gates_fwd_kernel");
  return FML_OK;
}

int32_t fml_lstm_bwd(fml_ctx* ctx, const fml_lstm_desc* d, const float* dh_last, float* dW, float* db, float* dx,
                     float* scratch) {
  FML_REQUIRE(ctx, d && dh_last && dW && db && scratch, "fml_lstm_bwd: NULL buffer");
  const int T = d->T, B = d->B, I = d->I, H = d->H, Z = H + I;
  const long long bh = (long long)B * H, b4h = (long long)B * 4 * H;
  float* dpre = scratch;                 // [T*B][4H]
  float* dh = scratch + (long long)T * b4h;  // [B][H]
  float* dc = dh + bh;                   // [B][H]
  FML_CUDA(ctx, cudaMemcpyAsync(dh, dh_last, bh * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  FML_CUDA(ctx, cudaMemsetAsync(dc, 0, bh * 4, ctx->stream));
  int32_t rc;
  for (int t = T - 1; t >= 0; t--) {
    lstm_gates_bwd_kernel<<<blocks_for(ctx, bh), 256, 0, ctx->stream>>>(dh, dc, d->gates + t * b4h, d->cells + t * bh,
                                                                        d->cells + (t + 1) * bh, dpre + t * b4h, B, H);
    if (t > 0) {
      // dh_{t-1} = dpre_t . Wh   (Wh = columns 0..H-1 of W)
      fml_gemm_desc r = gemm_defaults();
      r.M = B; r.N = H; r.K = 4 * H;
      r.A = dpre + t * b4h; r.lda = 4 * H;
      r.B = d->W; r.ldb = Z;
      r.C = dh; r.ldc = H;
      if ((rc = fml_gemm(ctx, &r))) return rc;
    }
  }
  FML_LAUNCH_CHECK(ctx, "lstm_gates_bwd_kernel");
  // dW[:, 0:H] += dpre^T . h_{t-1} over all steps; dW[:, H:] += dpre^T . x; db += column sums
  fml_gemm_desc wh = gemm_defaults();
  wh.M = 4 * H; wh.N = H; wh.K = T * B;
  wh.A = dpre; wh.lda = 4 * H; wh.transA = 1;
  wh.B = d->hs; wh.ldb = H;
  wh.C = dW; wh.ldc = Z; wh.beta = 1.f;
  if ((rc = fml_gemm(ctx, &wh))) return rc;
  fml_gemm_desc wx = gemm_defaults();
  wx.M = 4 * H; wx.N = I; wx.K = T * B;
  wx.A = dpre; wx.lda = 4 * H; wx.transA = 1;
  wx.B = d->x; wx.ldb = I;
  wx.C = dW + H; wx.ldc = Z; wx.beta = 1.f;
  if ((rc = fml_gemm(ctx, &wx))) return rc;
  if ((rc = fml_col_sum(ctx, dpre, db, (int64_t)T * B, 4 * H, 1))) return rc;
  if (dx) {
    fml_gemm_desc gx = gemm_defaults();
    gx.M = T * B; gx.N = I; gx.K = 4 * H;
    gx.A = dpre; gx.lda = 4 * H;
    gx.B = d->W + H; gx.ldb = Z;
    gx.C = dx; gx.ldc = I;
    if ((rc = fml_gemm(ctx, &gx))) return rc;
  }
  return FML_OK;
}

}  // extern "C"
