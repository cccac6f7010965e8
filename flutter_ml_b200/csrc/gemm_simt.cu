// CUDA-core fp32 contraction for shapes the tensor-core path cannot take (unaligned leading
// dimensions such as the 10-wide MLP head) and for FML_PREC_FP32.  64x64 output tile, 16-deep
// k slices, 256 threads with a 4x4 register block each; operands are addressed through
// generic (row, col) strides so all four transpose combinations share one kernel.
#include <algorithm>

#include "common.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

struct SimtParams {
  int M, N, K;
  const float* A; long long a_ri, a_rk;  // op(A)(i,k) = A[i*a_ri + k*a_rk]
  const float* B; long long b_rk, b_rj;  // op(B)(k,j) = B[k*b_rk + j*b_rj]
  float* C; float* Z; const float* bias;
  long long ldc;
  int nb1;
  long long sA1, sA2, sB1, sB2, sC1, sC2;
  int act; float alpha, beta;
  const float* dact_saved; int dact;
  int ksplit, kslice;  // ksplit > 1: blockIdx.z walks k slices of an unbatched product and the sums are added with atomics
};

__global__ void __launch_bounds__(256) gemm_simt_kernel(const SimtParams p) {
  __shared__ float As[TK][TM + 1];
  __shared__ float Bs[TK][TN + 1];
  const int b = p.ksplit > 1 ? 0 : blockIdx.z, b1 = b % p.nb1, b2 = b / p.nb1;
  const int kbeg = p.ksplit > 1 ? blockIdx.z * p.kslice : 0;
  const int kend = p.ksplit > 1 ? min(p.K, kbeg + p.kslice) : p.K;
  const float* A = p.A + b1 * p.sA1 + b2 * p.sA2;
  const float* B = p.B + b1 * p.sB1 + b2 * p.sB2;
  const long long coff = b1 * p.sC1 + b2 * p.sC2;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = kbeg; k0 < kend; k0 += TK) {
    for (int e = threadIdx.x; e < TM * TK; e += 256) {
      // consecutive threads walk the contiguous direction of the stored operand
      int i, k;
      if (p.a_rk == 1) { k = e % TK; i = e / TK; } else { i = e % TM; k = e / TM; }
      float v = 0.f;
      if (m0 + i < p.M && k0 + k < kend) v = A[(long long)(m0 + i) * p.a_ri + (long long)(k0 + k) * p.a_rk];
      As[k][i] = v;
    }
    for (int e = threadIdx.x; e < TN * TK; e += 256) {
      int j, k;
      if (p.b_rj == 1) { j = e % TN; k = e / TN; } else { k = e % TK; j = e / TK; }
      float v = 0.f;
      if (n0 + j < p.N && k0 + k < kend) v = B[(long long)(k0 + k) * p.b_rk + (long long)(n0 + j) * p.b_rj];
      Bs[k][j] = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; k++) {
      float a[4], bb[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = As[k][ty + 16 * i];
#pragma unroll
      for (int j = 0; j < 4; j++) bb[j] = Bs[k][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int row = m0 + ty + 16 * i;
    if (row >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int col = n0 + tx + 16 * j;
      if (col >= p.N) continue;
      const long long o = coff + (long long)row * p.ldc + col;
      if (p.ksplit > 1) {   // the host zeroed C when beta is 0; no epilogue extras in this mode
        atomicAdd(p.C + o, acc[i][j] * p.alpha);
        continue;
      }
      float v = acc[i][j] * p.alpha + (p.bias ? p.bias[col] : 0.f);
      if (p.Z) p.Z[o] = v;
      v = fml_act_apply(p.act, v);
      if (p.dact_saved) v *= fml_act_grad_small(p.dact, p.dact_saved[o]);
      if (p.beta != 0.f) v += p.C[o];
      p.C[o] = v;
    }
  }
}

}  // namespace

int32_t fml_gemm_simt(fml_ctx* ctx, const fml_gemm_desc* d) {
  SimtParams p;
  p.M = d->M; p.N = d->N; p.K = d->K;
  p.A = d->A; p.B = d->B; p.C = d->C; p.Z = d->preact; p.bias = d->bias;
  if (d->transA) { p.a_ri = 1; p.a_rk = d->lda; } else { p.a_ri = d->lda; p.a_rk = 1; }
  if (d->transB) { p.b_rk = 1; p.b_rj = d->ldb; } else { p.b_rk = d->ldb; p.b_rj = 1; }
  p.ldc = d->ldc;
  const int nb1 = d->batch1 < 1 ? 1 : d->batch1, nb2 = d->batch2 < 1 ? 1 : d->batch2;
  p.nb1 = nb1;
  p.sA1 = d->sA1; p.sA2 = d->sA2; p.sB1 = d->sB1; p.sB2 = d->sB2; p.sC1 = d->sC1; p.sC2 = d->sC2;
  p.act = d->act; p.alpha = d->alpha; p.beta = d->beta;
  p.dact_saved = d->dact_saved; p.dact = d->dact;
  FML_REQUIRE(ctx, (long long)nb1 * nb2 <= 65535, "fml_gemm: more than 65535 batches on the CUDA-core path");
  dim3 grid((d->N + TN - 1) / TN, (d->M + TM - 1) / TM, nb1 * nb2);
  FML_REQUIRE(ctx, grid.y <= 65535, "fml_gemm: M too large for the CUDA-core path");
  // A few output tiles under a long k (the weight gradient of a narrow layer over a large batch: 64 x 10 outputs,
  // k = batch rows) would run on one or two SMs: cut k into slices, one block each, summed with atomics.
  p.ksplit = 1;
  p.kslice = d->K;
  const long long tiles = (long long)grid.x * grid.y;
  if (nb1 * nb2 == 1 && !d->bias && !d->preact && d->act == FML_ACT_NONE && !d->dact_saved && d->K >= 2048 &&
      tiles * 2 <= ctx->sm_count) {
    int ks = (int)std::min<long long>(2ll * ctx->sm_count / tiles, d->K / 256);
    ks = std::min(ks, 65535);
    if (ks > 1) {
      p.kslice = (((d->K + ks - 1) / ks) + TK - 1) / TK * TK;
      p.ksplit = (d->K + p.kslice - 1) / p.kslice;
      grid.z = p.ksplit;
      if (d->beta == 0.f)
        FML_CUDA(ctx, cudaMemset2DAsync(d->C, (size_t)d->ldc * 4, 0, (size_t)d->N * 4, (size_t)d->M, ctx->stream));
    }
  }
  gemm_simt_kernel<<<grid, 256, 0, ctx->stream>>>(p);
  FML_LAUNCH_CHECK(ctx, "gemm_simt_kernel");
  ctx->last_gemm_path = 2;
  ctx->last_gemm_tile[0] = ctx->last_gemm_tile[1] = ctx->last_gemm_tile[2] = ctx->last_gemm_tile[3] = 0;
  return FML_OK;
}
