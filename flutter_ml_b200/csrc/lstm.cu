// LSTM layer over a batch of sequences.  The four gate matrices are regrouped so that the gates of
// one hidden unit are adjacent rows ("gate-interleaved"); then
//   - the input projection of ALL timesteps is one large GEMM (bias in its epilogue);
//   - each timestep is ONE tensor-core GEMM h_{t-1}.Wh^T whose epilogue adds the input projection,
//     applies the four gate nonlinearities and the cell update, and writes gates, c_t and h_t
//     (a thread owns one batch row and 32 consecutive columns = 8 hidden units x 4 gates);
//   - BPTT is ONE fused launch per step in TF32 mode (gate derivatives + product + sum over the K split,
//     lstm_bwd_tc.cu; other modes and shapes: one gate-gradient kernel and one small split-K GEMM per step), then the
//     weight gradients of all timesteps as two large GEMMs, regrouped back to the reference's row order.
// Saved gates are [T][B][H][4] (f, i, c~, o per hidden unit).
//
// Reference: LSTMLayer.forward lib/layertypes/lstmLayer.dart:112-150.  Gate order f,i,c~,o
// (:64); weight columns [h_{t-1} | x_t] (:119).
#include <stdlib.h>

#include <algorithm>

#include "common.cuh"

// the recurrence of all time steps in one cooperative kernel (lstm_tc.cu); 1 = shape not eligible
int32_t fml_lstm_fwd_persistent(fml_ctx* ctx, const fml_lstm_desc* d, const float* Wi, int fast_math);
// the backward recurrence of all time steps in one cooperative kernel (lstm_bwd_tc.cu); 1 = not eligible / launch refused
int32_t fml_lstm_bwd_persistent(fml_ctx* ctx, const fml_lstm_desc* d, const float* Wi, const float* dh_last, float* dpre,
                                float* dh_a, float* dh_b);
// steps T-1 .. 1 of the backward recurrence as one fused launch per step (lstm_bwd_tc.cu); 1 = shape not eligible
int32_t fml_lstm_bwd_steps(fml_ctx* ctx, const fml_lstm_desc* d, const float* Wi, const float* dh_last, float* dpre, float* work,
                           float** dh_final, float** dc_final);

namespace {

// W' = W with rows regrouped so that the four gates of a hidden unit are adjacent:
// W'[4*r + q][:] = W[q*H + r][:]   (reference order: gate-major, lstmLayer.dart:64)
__global__ void lstm_interleave_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, int H, int Z) {
  const long long n = 4ll * H * Z;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % Z);
    const int row = (int)(i / Z);  // destination row 4*r + q
    const int r = row >> 2, q = row & 3;
    dst[i] = src[((long long)q * H + r) * Z + c];
  }
}
// dst[q*H + r][:] += src[4*r + q][:]  (gradients back into the reference's row order)
__global__ void lstm_deinterleave_add_kernel(const float* __restrict__ src, float* __restrict__ dst, int H, int Z) {
  const long long n = 4ll * H * Z;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % Z);
    const int row = (int)(i / Z);
    const int r = row >> 2, q = row & 3;
    dst[((long long)q * H + r) * Z + c] += src[i];
  }
}

// Fallback gate kernel (CUDA-core path, shapes the tensor-core epilogue cannot take): pre [B][4H]
// gate-interleaved -> activated gates, c_t, h_t
__global__ void lstm_gates_fwd_kernel(const float* __restrict__ pre, const float* __restrict__ c_prev,
                                      float* __restrict__ gates, float* __restrict__ c_out, float* __restrict__ h_out,
                                      int B, int H) {
  const int n = B * H;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += gridDim.x * blockDim.x) {
    const float4 p = reinterpret_cast<const float4*>(pre)[idx];
    const float f = fml_sigmoid(p.x), i = fml_sigmoid(p.y), g = fml_tanh_ref(p.z), o = fml_sigmoid(p.w);
    const float c = f * c_prev[idx] + i * g;
    reinterpret_cast<float4*>(gates)[idx] = make_float4(f, i, g, o);
    c_out[idx] = c;
    h_out[idx] = o * fml_tanh_ref(c);
  }
}

// dh, dc (in/out: becomes dc_{t-1}), saved gates (interleaved) and cells -> gradient of the pre-activations
__global__ void lstm_gates_bwd_kernel(float* __restrict__ dh, float* dc, const float* __restrict__ gates,
                                      const float* __restrict__ c_prev, const float* __restrict__ c_cur,
                                      float* __restrict__ dpre, int B, int H) {
  // The recurrent product queued behind this kernel may set up (barriers, TMEM) while this one runs, and this kernel
  // itself is launched while the previous product drains.  What does not depend on that product (the saved gates and
  // cells of this step, a DRAM round trip) is loaded BEFORE the wait for it; only dh and dc are read after.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int n = B * H;
  const int stride = gridDim.x * blockDim.x;
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  float4 gt = make_float4(0.f, 0.f, 0.f, 0.f);
  float cc = 0.f, cp = 0.f;
  if (idx < n) {
    gt = __ldg(reinterpret_cast<const float4*>(gates) + idx);
    cc = __ldg(c_cur + idx);
    cp = __ldg(c_prev + idx);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (; idx < n; idx += stride) {
    const float f = gt.x, i = gt.y, g = gt.z, o = gt.w;
    const float tc = fml_tanh_ref(cc);
    const float dhv = dh[idx];
    dh[idx] = 0.f;  // the product that follows ADDS dpre_t . Wh into dh (its K-split partial sums need a zeroed target)
    const float d_o = dhv * tc;
    const float dct = dc[idx] + dhv * o * (1.f - tc * tc);
    reinterpret_cast<float4*>(dpre)[idx] = make_float4(dct * cp * (f * (1.f - f)), dct * g * (i * (1.f - i)), dct * i * (1.f - g * g),
                                                       d_o * (o * (1.f - o)));
    dc[idx] = dct * f;
    const int nx = idx + stride;   // grids smaller than B*H (very large batches): the next element's inputs
    if (nx < n) {
      gt = __ldg(reinterpret_cast<const float4*>(gates) + nx);
      cc = __ldg(c_cur + nx);
      cp = __ldg(c_prev + nx);
    }
  }
}

// One cell update on pre-activations the CALLER formed (the tiered layers, lib/layertypes/multilstm.dart:160-178): gate
// blocks f | i | c~ | o, column g*H + u of a [B][4H] row, the order of the reference's four weight matrices stacked.
__global__ void lstm_cell_fwd_kernel(const float* __restrict__ pre, const float* __restrict__ c_prev, float* __restrict__ gates,
                                     float* __restrict__ c_out, float* __restrict__ h_out, int B, int H) {
  const int n = B * H;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += gridDim.x * blockDim.x) {
    const int b = idx / H, u = idx - b * H;
    const float* pr = pre + (long long)b * 4 * H + u;
    float* gr = gates + (long long)b * 4 * H + u;
    const float f = fml_sigmoid(pr[0]), i = fml_sigmoid(pr[H]), g = fml_tanh_ref(pr[2 * H]), o = fml_sigmoid(pr[3 * H]);
    const float c = f * c_prev[idx] + i * g;
    gr[0] = f; gr[H] = i; gr[2 * H] = g; gr[3 * H] = o;
    c_out[idx] = c;
    h_out[idx] = o * fml_tanh_ref(c);
  }
}

// dh and (optionally) dc flowing into the cell from later steps -> gradient of the pre-activations and of c_prev; the
// derivatives are formed from the saved outputs as in the reference (sigmoid y(1-y) tensor.dart:552, tanh 1-y^2 :598)
__global__ void lstm_cell_bwd_kernel(const float* __restrict__ gates, const float* __restrict__ c_prev, const float* __restrict__ c_cur,
                                     const float* __restrict__ dh, const float* __restrict__ dc_in, float* __restrict__ dpre,
                                     float* __restrict__ dc_prev, int accumulate_dc_prev, int B, int H) {
  const int n = B * H;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += gridDim.x * blockDim.x) {
    const int b = idx / H, u = idx - b * H;
    const float* gr = gates + (long long)b * 4 * H + u;
    float* dp = dpre + (long long)b * 4 * H + u;
    const float f = gr[0], i = gr[H], g = gr[2 * H], o = gr[3 * H];
    const float tc = fml_tanh_ref(c_cur[idx]);
    const float dhv = dh ? dh[idx] : 0.f;
    const float dct = (dc_in ? dc_in[idx] : 0.f) + dhv * o * (1.f - tc * tc);
    dp[0] = dct * c_prev[idx] * (f * (1.f - f));
    dp[H] = dct * g * (i * (1.f - i));
    dp[2 * H] = dct * i * (1.f - g * g);
    dp[3 * H] = dhv * tc * (o * (1.f - o));
    const float v = dct * f;
    dc_prev[idx] = accumulate_dc_prev ? dc_prev[idx] + v : v;
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

// stream-ordered temporary (freed with cudaFreeAsync by the caller)
int32_t temp_alloc(fml_ctx* ctx, size_t n_floats, float** out) {
  cudaError_t e = cudaMallocAsync(reinterpret_cast<void**>(out), n_floats * sizeof(float), ctx->stream);
  if (e != cudaSuccess) return fml_fail(ctx, FML_ERR_OOM, std::string("lstm temporary: ") + cudaGetErrorString(e));
  return FML_OK;
}

}  // namespace

extern "C" {

int32_t fml_lstm_fwd(fml_ctx* ctx, const fml_lstm_desc* d) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, d && d->W && d->b && d->x && d->gates && d->cells && d->hs && d->xproj, "fml_lstm_fwd: NULL buffer");
  FML_REQUIRE(ctx, d->T > 0 && d->B > 0 && d->I > 0 && d->H > 0, "fml_lstm_fwd: bad sizes");
  const int T = d->T, B = d->B, I = d->I, H = d->H, Z = H + I;
  const long long bh = (long long)B * H, b4h = (long long)B * 4 * H;
  FML_CUDA(ctx, cudaMemsetAsync(d->cells, 0, bh * 4, ctx->stream));
  FML_CUDA(ctx, cudaMemsetAsync(d->hs, 0, bh * 4, ctx->stream));
  // gate-interleaved copies of W and b: the four gates of a hidden unit become adjacent columns of every product
  float* Wi = nullptr;
  int32_t rc = temp_alloc(ctx, (size_t)4 * H * Z + 4 * H, &Wi);
  if (rc) return rc;
  float* bi = Wi + (size_t)4 * H * Z;
  lstm_interleave_rows_kernel<<<blocks_for(ctx, 4ll * H * Z), 256, 0, ctx->stream>>>(d->W, Wi, H, Z);
  lstm_interleave_rows_kernel<<<blocks_for(ctx, 4ll * H), 256, 0, ctx->stream>>>(d->b, bi, H, 1);
  // xproj[T*B][4H] = x . Wx^T + b   (Wx = columns H.. of W), all timesteps in one product
  fml_gemm_desc g = gemm_defaults();
  g.M = T * B; g.N = 4 * H; g.K = I;
  g.A = d->x; g.lda = I;
  g.B = Wi + H; g.ldb = Z; g.transB = 1;
  g.C = d->xproj; g.ldc = 4 * H;
  g.bias = bi;
  rc = fml_gemm(ctx, &g);
  const int prec = ctx->precision;
  {
    static int persistent = -1;
    if (persistent < 0) {
      const char* e = getenv("FML_LSTM_PERSISTENT");   // diagnostics: 0 keeps the per-step kernels
      persistent = e ? atoi(e) : 1;
    }
    if (rc == FML_OK && persistent && prec == FML_PREC_TF32) {
      const int32_t pr = fml_lstm_fwd_persistent(ctx, d, Wi, 1);
      if (pr <= 0) {   // done, or failed for good
        cudaFreeAsync(Wi, ctx->stream);
        return pr;
      }
    }
  }
  for (int t = 0; t < T && rc == FML_OK; t++) {
    float* pre = d->xproj + t * b4h;
    fml_gemm_desc r = gemm_defaults();
    r.M = B; r.N = 4 * H; r.K = H;
    r.A = d->hs + t * bh; r.lda = H;
    r.B = Wi; r.ldb = Z; r.transB = 1;
    r.C = pre; r.ldc = 4 * H; r.beta = 1.f;
    const bool fused = prec != FML_PREC_FP32 && fml_gemm_tc_eligible(&r) && (H % 8 == 0) &&
                       (reinterpret_cast<uintptr_t>(pre) & 15) == 0;
    if (fused) {
      // recurrent product with the gate nonlinearity and the cell update in its epilogue
      fml_lstm_epilogue le = {pre, d->cells + t * bh, d->cells + (t + 1) * bh, d->hs + (t + 1) * bh, d->gates + t * b4h,
                              prec == FML_PREC_TF32 ? 1 : 0};
      r.beta = 0.f;
      rc = fml_gemm_tc(ctx, &r, prec, &le);
    } else {
      if (t > 0) rc = fml_gemm(ctx, &r);
      if (rc == FML_OK)
        lstm_gates_fwd_kernel<<<blocks_for(ctx, bh), 256, 0, ctx->stream>>>(pre, d->cells + t * bh, d->gates + t * b4h,
                                                                            d->cells + (t + 1) * bh, d->hs + (t + 1) * bh, B, H);
    }
  }
  cudaFreeAsync(Wi, ctx->stream);
  if (rc) return rc;
  FML_LAUNCH_CHECK(ctx, "lstm forward");
  return FML_OK;
}

int32_t fml_lstm_bwd(fml_ctx* ctx, const fml_lstm_desc* d, const float* dh_last, float* dW, float* db, float* dx,
                     float* scratch) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, d && dh_last && dW && db && scratch, "fml_lstm_bwd: NULL buffer");
  const int T = d->T, B = d->B, I = d->I, H = d->H, Z = H + I;
  const long long bh = (long long)B * H, b4h = (long long)B * 4 * H;
  float* dpre = scratch;                     // [T*B][4H], gate-interleaved
  float* dh = scratch + (long long)T * b4h;  // [B][H]
  float* dc = dh + bh;                       // [B][H]
  // temporaries: interleaved W, interleaved dW and db
  float* Wi = nullptr;
  int32_t rc = temp_alloc(ctx, (size_t)2 * 4 * H * Z + 4 * H, &Wi);
  if (rc) return rc;
  float* dWi = Wi + (size_t)4 * H * Z;
  float* dbi = dWi + (size_t)4 * H * Z;
  lstm_interleave_rows_kernel<<<blocks_for(ctx, 4ll * H * Z), 256, 0, ctx->stream>>>(d->W, Wi, H, Z);
  cudaMemsetAsync(dWi, 0, ((size_t)4 * H * Z + 4 * H) * sizeof(float), ctx->stream);
  bool recurrence_done = false;
  {
    // Opt-in (FML_LSTM_BWD_SINGLE_KERNEL=1, read at every call): the whole recurrence as one cooperative kernel that sums
    // the split contraction in a fixed order, so dpre, dW, db come out bit for bit the same on every run.  It is NOT the
    // default because it is slower than the launch per step below (24 us against 8 us per step at H 512, B 128:
    // measured phase by phase, see lstm_bwd_tc.cu), which sums the K split's partial tiles in no fixed order.
    const char* e = getenv("FML_LSTM_BWD_SINGLE_KERNEL");
    if (e && atoi(e) != 0 && ctx->precision == FML_PREC_TF32) {
      const int32_t pr = fml_lstm_bwd_persistent(ctx, d, Wi, dh_last, dpre, dh, dc);   // dh, dc: its two dh buffers
      if (pr < 0) {
        cudaFreeAsync(Wi, ctx->stream);
        return pr;
      }
      recurrence_done = pr == 0;
    }
  }
  // Default for TF32 at batch <= 128 and H in {128, 256, 384, 512}: one fused launch per step (gate derivatives, product
  // and the sum over the K split in one kernel, consecutive steps chained by programmatic dependent launch);
  // FML_LSTM_BWD_FUSED=0 keeps the gate kernel + K-split product per step below (diagnostics, read at every call).
  int t_first = T - 1;
  float* work = nullptr;
  if (!recurrence_done && ctx->precision == FML_PREC_TF32) {
    const char* e = getenv("FML_LSTM_BWD_FUSED");
    if (!(e && atoi(e) == 0)) {
      rc = temp_alloc(ctx, (size_t)5 * bh, &work);
      if (rc) {
        cudaFreeAsync(Wi, ctx->stream);
        return rc;
      }
      float *dh_f = nullptr, *dc_f = nullptr;
      const int32_t pr = fml_lstm_bwd_steps(ctx, d, Wi, dh_last, dpre, work, &dh_f, &dc_f);
      if (pr < 0) {
        cudaFreeAsync(work, ctx->stream);
        cudaFreeAsync(Wi, ctx->stream);
        return pr;
      }
      if (pr == 0) {   // only dpre_0 is left: the gate kernel on the buffers the chain ended in
        dh = dh_f;
        dc = dc_f;
        t_first = 0;
      }
    }
  }
  if (!recurrence_done && t_first == T - 1) {
    cudaMemcpyAsync(dh, dh_last, bh * 4, cudaMemcpyDeviceToDevice, ctx->stream);
    cudaMemsetAsync(dc, 0, bh * 4, ctx->stream);
  }
  for (int t = t_first; t >= 0 && rc == FML_OK && !recurrence_done; t--) {
    {
      cudaLaunchConfig_t cfg = {};
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.gridDim = dim3(blocks_for(ctx, bh));
      cfg.blockDim = dim3(256);
      cfg.stream = ctx->stream;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      FML_CUDA(ctx, cudaLaunchKernelEx(&cfg, lstm_gates_bwd_kernel, dh, dc, (const float*)(d->gates + t * b4h),
                                       (const float*)(d->cells + t * bh), (const float*)(d->cells + (t + 1) * bh),
                                       dpre + t * b4h, B, H));
    }
    if (t > 0) {
      // dh_{t-1} = dpre_t . Wh   (Wh = columns 0..H-1 of the interleaved W)
      fml_gemm_desc r = gemm_defaults();
      r.M = B; r.N = H; r.K = 4 * H;
      r.A = dpre + t * b4h; r.lda = 4 * H;
      r.B = Wi; r.ldb = Z;
      r.C = dh; r.ldc = H; r.beta = 1.f;  // dh was zeroed by the gate kernel above
      rc = fml_gemm(ctx, &r);
    }
  }
  // dW'[:, 0:H] = dpre^T . h_{t-1} over all steps; dW'[:, H:] = dpre^T . x; db' = column sums
  if (rc == FML_OK) {
    fml_gemm_desc wh = gemm_defaults();
    wh.M = 4 * H; wh.N = H; wh.K = T * B;
    wh.A = dpre; wh.lda = 4 * H; wh.transA = 1;
    wh.B = d->hs; wh.ldb = H;
    wh.C = dWi; wh.ldc = Z; wh.beta = 1.f;
    rc = fml_gemm(ctx, &wh);
  }
  if (rc == FML_OK) {
    fml_gemm_desc wx = gemm_defaults();
    wx.M = 4 * H; wx.N = I; wx.K = T * B;
    wx.A = dpre; wx.lda = 4 * H; wx.transA = 1;
    wx.B = d->x; wx.ldb = I;
    wx.C = dWi + H; wx.ldc = Z; wx.beta = 1.f;
    rc = fml_gemm(ctx, &wx);
  }
  if (rc == FML_OK) rc = fml_col_sum(ctx, dpre, dbi, (int64_t)T * B, 4 * H, 1);
  if (rc == FML_OK) {
    // back to the reference's gate-major row order, accumulating like every gradient
    lstm_deinterleave_add_kernel<<<blocks_for(ctx, 4ll * H * Z), 256, 0, ctx->stream>>>(dWi, dW, H, Z);
    lstm_deinterleave_add_kernel<<<blocks_for(ctx, 4ll * H), 256, 0, ctx->stream>>>(dbi, db, H, 1);
  }
  if (rc == FML_OK && dx) {
    fml_gemm_desc gx = gemm_defaults();
    gx.M = T * B; gx.N = I; gx.K = 4 * H;
    gx.A = dpre; gx.lda = 4 * H;
    gx.B = Wi + H; gx.ldb = Z;
    gx.C = dx; gx.ldc = I;
    rc = fml_gemm(ctx, &gx);
  }
  if (work) cudaFreeAsync(work, ctx->stream);
  cudaFreeAsync(Wi, ctx->stream);
  if (rc) return rc;
  FML_LAUNCH_CHECK(ctx, "lstm backward");
  return FML_OK;
}

int32_t fml_lstm_cell_fwd(fml_ctx* ctx, const float* pre, const float* c_prev, float* gates, float* c, float* h, int64_t B, int64_t H) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, pre && c_prev && gates && c && h, "fml_lstm_cell_fwd: NULL buffer");
  FML_REQUIRE(ctx, B > 0 && H > 0 && B * H <= 0x7fffffffLL / 4, "fml_lstm_cell_fwd: bad sizes");
  lstm_cell_fwd_kernel<<<blocks_for(ctx, B * H), 256, 0, ctx->stream>>>(pre, c_prev, gates, c, h, (int)B, (int)H);
  FML_LAUNCH_CHECK(ctx, "lstm_cell_fwd_kernel");
  return FML_OK;
}

int32_t fml_lstm_cell_bwd(fml_ctx* ctx, const float* gates, const float* c_prev, const float* c, const float* dh, const float* dc,
                          float* dpre, float* dc_prev, int32_t accumulate_dc_prev, int64_t B, int64_t H) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, gates && c_prev && c && dpre && dc_prev, "fml_lstm_cell_bwd: NULL buffer");
  FML_REQUIRE(ctx, B > 0 && H > 0 && B * H <= 0x7fffffffLL / 4, "fml_lstm_cell_bwd: bad sizes");
  lstm_cell_bwd_kernel<<<blocks_for(ctx, B * H), 256, 0, ctx->stream>>>(gates, c_prev, c, dh, dc, dpre, dc_prev, accumulate_dc_prev ? 1 : 0,
                                                                        (int)B, (int)H);
  FML_LAUNCH_CHECK(ctx, "lstm_cell_bwd_kernel");
  return FML_OK;
}

}  // extern "C"
