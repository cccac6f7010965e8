// Tape executor: runs a caller-supplied list of autograd nodes forward or backward with one call.
//
// The reference builds a graph of Node{inputs, backwardFn, opName, extraParams}
// (lib/autogradEngine/tensor.dart:5-19) and Tensor.backward (tensor.dart:43-75) topologically sorts it and
// calls the closures last to first; every closure ADDS into the gradients of its inputs.  Here the host
// describes each node as an fml_op (kind = the opName, device buffers instead of nested lists) and the whole
// sweep is enqueued on the context's stream: contractions go to fml_gemm (beta = 1 gives the += of
// tensor.dart:918-941), the rest to the streaming kernels of this library or to the small accumulate-form
// kernels below.  Nothing here allocates besides the context's scratch arena, so a sweep can be recorded
// into a CUDA graph.
#include <cstring>

#include "common.cuh"

namespace {

constexpr int TP_THREADS = 256;
inline int tp_blocks(fml_ctx* ctx, long long n) {
  long long b = (n + TP_THREADS - 1) / TP_THREADS;
  return (int)std::max<long long>(1, std::min<long long>(b, (long long)ctx->sm_count * 8));
}
#define TP_LOOP(i, n) \
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (n); i += (long long)gridDim.x * blockDim.x)

// gin += g * other   (elementWiseMultiply backward, tensor.dart:486-491)
__global__ void mul_acc_kernel(const float* __restrict__ g, const float* __restrict__ other, float* gin, long long n) {
  TP_LOOP(i, n) gin[i] += g[i] * other[i];
}
// y += s[0] * c * x   (a gradient rule whose upstream is a device scalar)
__global__ void scaled_add_dev_kernel(float* y, const float* __restrict__ x, const float* __restrict__ s, float c, long long n) {
  const float k = s[0] * c;
  TP_LOOP(i, n) y[i] += k * x[i];
}
// gin += gout[0] * k * (p - t)   (mse / mseMatrix backward, tensor.dart:507-512, 994-1003)
__global__ void mse_bwd_kernel(const float* __restrict__ p, const float* __restrict__ t, const float* __restrict__ gout,
                               float* gin, float k, long long n) {
  const float kk = gout[0] * k;
  TP_LOOP(i, n) gin[i] += kk * (p[i] - t[i]);
}
// gin += gout[0]   (sum / sumMatrix backward, tensor.dart:569-573)
__global__ void broadcast_add_dev_kernel(float* gin, const float* __restrict__ gout, long long n) {
  const float g = gout[0];
  TP_LOOP(i, n) gin[i] += g;
}
// out = in + s[0]   (addScalarToMatrix, tensor.dart:711-723)
__global__ void add_scalar_dev_kernel(const float* __restrict__ in, const float* __restrict__ s, float* __restrict__ out, long long n) {
  const float v = s[0];
  TP_LOOP(i, n) out[i] = in[i] + v;
}
__global__ void add_one_dev_kernel(float* y, const float* __restrict__ x) { y[0] += x[0]; }
// part[r][c] += whole[r][off + c]   (concat backward, tensor.dart:443-449, 749-757)
__global__ void split_add_kernel(float* part, const float* __restrict__ whole, long long rows, int pc, int ld, int off) {
  TP_LOOP(i, rows * pc) {
    const long long r = i / pc;
    const int c = (int)(i - r * pc);
    part[i] += whole[r * ld + off + c];
  }
}
// out[c][r] += in[r][c] through a padded shared tile (transpose backward, tensor.dart:1222-1228)
__global__ void transpose_acc_kernel(const float* __restrict__ in, float* out, long long rows, long long cols) {
  __shared__ float tile[32][33];
  const long long r0 = (long long)blockIdx.y * 32, c0 = (long long)blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int j = ty; j < 32; j += 8)
    if (r0 + j < rows && c0 + tx < cols) tile[j][tx] = in[(r0 + j) * cols + c0 + tx];
  __syncthreads();
  for (int j = ty; j < 32; j += 8)
    if (c0 + j < cols && r0 + tx < rows) out[(c0 + j) * rows + r0 + tx] += tile[tx][j];
}

// Sum of n floats: per-block double partials, then one block folds them (sum / sumMatrix, tensor.dart:561-567).
__global__ void __launch_bounds__(TP_THREADS) sum_partial_kernel(const float* __restrict__ x, double* __restrict__ partial, long long n) {
  __shared__ double red[TP_THREADS / 32];
  double acc = 0.0;
  TP_LOOP(i, n) acc += (double)x[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < TP_THREADS / 32; w++) t += red[w];
    partial[blockIdx.x] = t;
  }
}
__global__ void __launch_bounds__(TP_THREADS) sum_final_kernel(const double* __restrict__ partial, int n, float* out) {
  __shared__ double red[TP_THREADS / 32];
  double acc = 0.0;
  for (int i = threadIdx.x; i < n; i += TP_THREADS) acc += partial[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < TP_THREADS / 32; w++) t += red[w];
    out[0] = (float)t;
  }
}

// ---- matrix-vector kernels: every element of the matrix is read (or updated) exactly once -------------------
// y[i] = sum_j W[i][j] x[j]: one warp per row, 128-bit loads when the row pitch allows (tensor.dart:956-960)
__global__ void __launch_bounds__(TP_THREADS) gemv_kernel(const float* __restrict__ W, const float* __restrict__ x,
                                                          float* __restrict__ y, int rows, int cols, int vec) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const float* w = W + (size_t)r * cols;
    float acc = 0.f;
    if (vec) {
      const float4* w4 = reinterpret_cast<const float4*>(w);
      const float4* x4 = reinterpret_cast<const float4*>(x);
      for (int j = lane; j < (cols >> 2); j += 32) {
        const float4 a = w4[j], b = x4[j];
        acc += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
      }
    } else {
      for (int j = lane; j < cols; j += 32) acc += w[j] * x[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) y[r] = acc;
  }
}
// dW[i][j] += dy[i] * x[j]  and  dx[j] += sum_i W[i][j] dy[i]  in one pass over a block of rows
// (the two loops of the matVecMul closure, tensor.dart:965-974).  Grid: (column tiles of 256, row chunks).
__global__ void __launch_bounds__(TP_THREADS) gemv_bwd_kernel(const float* __restrict__ W, const float* __restrict__ x,
                                                              const float* __restrict__ dy, float* dW, float* dx,
                                                              int rows, int cols, int rows_per_block) {
  const int j = blockIdx.x * TP_THREADS + threadIdx.x;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  if (j >= cols) return;
  const float xj = dW ? x[j] : 0.f;
  float acc = 0.f;
  for (int r = r0; r < r1; r++) {
    const float g = dy[r];
    const size_t idx = (size_t)r * cols + j;
    if (dx) acc += W[idx] * g;
    if (dW) dW[idx] += g * xj;
  }
  if (dx) atomicAdd(dx + j, acc);
}

}  // namespace

namespace {

int32_t tp_gemm(fml_ctx* ctx, const float* A, const float* B, float* C, int M, int N, int K, bool tA, bool tB, float beta,
                int prec, const float* bias = nullptr, float* preact = nullptr, int act = FML_ACT_NONE) {
  fml_gemm_desc d;
  std::memset(&d, 0, sizeof(d));
  d.M = M; d.N = N; d.K = K;
  d.transA = tA; d.transB = tB;
  d.lda = tA ? M : K; d.ldb = tB ? K : N; d.ldc = N;
  d.A = A; d.B = B; d.C = C;
  d.bias = bias; d.preact = preact; d.act = act;
  d.alpha = 1.f; d.beta = beta;
  d.batch1 = d.batch2 = 1;
  d.precision = prec;
  return fml_gemm(ctx, &d);
}

inline bool al16p(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int act_of_kind(int kind) {
  switch (kind) {
    case FML_OP_RELU: return FML_ACT_RELU;
    case FML_OP_SIGMOID: return FML_ACT_SIGMOID;
    case FML_OP_TANH: return FML_ACT_TANH;
    case FML_OP_GELU: return FML_ACT_GELU;
    default: return FML_ACT_NONE;
  }
}
int act2_of_kind(int kind) {
  switch (kind) {
    case FML_OP_LEAKY_RELU: return FML_ACT2_LEAKY_RELU;
    case FML_OP_ELU: return FML_ACT2_ELU;
    case FML_OP_SWISH: return FML_ACT2_SWISH;
    default: return FML_ACT2_MISH;
  }
}

#define TP_TRY(call)          \
  do {                        \
    int32_t rc__ = (call);    \
    if (rc__) return rc__;    \
  } while (0)

int32_t attention_desc_of(fml_ctx* ctx, const fml_op& o, const std::string& where, fml_attention_desc* d) {
  FML_REQUIRE(ctx, o.in[0] && o.in[1] && o.in[2] && o.aux[0] && o.aux[1] && o.inner > 0 && o.rows % o.inner == 0 && o.cols % 64 == 0,
              where + " (attention): needs Q, K, V, aux[0], aux[1], rows = sequences * inner and cols = heads * 64");
  std::memset(d, 0, sizeof(*d));
  d->n_seq = o.rows / o.inner; d->seq_len = o.inner; d->heads = o.cols / 64; d->d_head = 64;
  d->q = o.in[0]; d->k = o.in[1]; d->v = o.in[2]; d->ld_qkv = o.cols;
  d->out = o.out; d->ld_out = o.cols; d->lse = o.aux[0];
  d->scale = o.s; d->causal = o.iparam != 0;
  return FML_OK;
}

int32_t op_forward(fml_ctx* ctx, const fml_op& o, int idx) {
  const long long n = (long long)o.rows * o.cols;
  const std::string where = "fml_tape_run: op " + std::to_string(idx);
  FML_REQUIRE(ctx, o.rows > 0 && o.cols > 0 && o.out, where + ": bad output shape or buffer");
  cudaStream_t st = ctx->stream;
  switch (o.kind) {
    case FML_OP_MATMUL:
      FML_REQUIRE(ctx, o.in[0] && o.in[1] && o.inner > 0, where + " (matMul): missing input");
      return tp_gemm(ctx, o.in[0], o.in[1], o.out, o.rows, o.cols, o.inner, false, false, 0.f, o.precision);
    case FML_OP_DENSE: {
      FML_REQUIRE(ctx, o.in[0] && o.in[1] && o.inner > 0, where + " (dense): missing input");
      FML_REQUIRE(ctx, o.iparam != FML_ACT_GELU || o.aux[0], where + " (dense): GELU needs aux[0] for the pre-activation");
      return tp_gemm(ctx, o.in[0], o.in[1], o.out, o.rows, o.cols, o.inner, false, false, 0.f, o.precision, o.in[2],
                     o.iparam == FML_ACT_GELU ? o.aux[0] : nullptr, o.iparam);
    }
    case FML_OP_MATVECMUL: {
      FML_REQUIRE(ctx, o.in[0] && o.in[1] && o.inner > 0 && o.rows == 1, where + " (matVecMul): missing input or rows != 1");
      const int vec = (o.inner % 4 == 0) && al16p(o.in[0]) && al16p(o.in[1]);
      const int blocks = std::max(1, std::min((o.cols + 7) / 8, ctx->sm_count * 8));
      gemv_kernel<<<blocks, TP_THREADS, 0, st>>>(o.in[0], o.in[1], o.out, o.cols, o.inner, vec);
      FML_LAUNCH_CHECK(ctx, "gemv_kernel");
      return FML_OK;
    }
    case FML_OP_ADD_MATRIX_AND_VECTOR:
      FML_REQUIRE(ctx, o.in[0] && o.in[1], where + " (addMatrixAndVector): missing input");
      return fml_add_bias(ctx, o.in[0], o.in[1], o.out, o.rows, o.cols);
    case FML_OP_ADD:
      FML_REQUIRE(ctx, o.in[0] && o.in[1], where + " (add): missing input");
      return fml_add(ctx, o.in[0], o.in[1], o.out, n);
    case FML_OP_MULTIPLY:
      FML_REQUIRE(ctx, o.in[0] && o.in[1], where + " (multiply): missing input");
      return fml_mul(ctx, o.in[0], o.in[1], o.out, n);
    case FML_OP_RELU: case FML_OP_SIGMOID: case FML_OP_TANH: case FML_OP_GELU:
      FML_REQUIRE(ctx, o.in[0], where + " (activation): missing input");
      return fml_act_fwd(ctx, act_of_kind(o.kind), o.in[0], o.out, n);
    case FML_OP_LEAKY_RELU: case FML_OP_ELU: case FML_OP_SWISH: case FML_OP_MISH:
      FML_REQUIRE(ctx, o.in[0], where + " (activation): missing input");
      return fml_act2_fwd(ctx, act2_of_kind(o.kind), o.s, o.in[0], o.out, n);
    case FML_OP_SCALE_MATRIX:
      FML_REQUIRE(ctx, o.in[0], where + " (scale_matrix): missing input");
      TP_TRY(fml_zero(ctx, o.out, n));
      return fml_axpy(ctx, o.s, o.in[0], o.out, n);
    case FML_OP_TRANSPOSE:
      FML_REQUIRE(ctx, o.in[0], where + " (transpose): missing input");
      return fml_transpose(ctx, o.in[0], o.out, o.cols, o.rows);  // in0 is cols x rows
    case FML_OP_CONCAT: {
      FML_REQUIRE(ctx, o.parts && o.part_cols && o.n_parts > 0, where + " (concat): missing parts");
      int off = 0;
      for (int p = 0; p < o.n_parts; p++) {
        const int pc = o.part_cols[p];
        FML_REQUIRE(ctx, o.parts[p] && pc > 0 && off + pc <= o.cols, where + " (concat): bad part");
        FML_CUDA(ctx, cudaMemcpy2DAsync(o.out + off, (size_t)o.cols * 4, o.parts[p], (size_t)pc * 4, (size_t)pc * 4,
                                        (size_t)o.rows, cudaMemcpyDeviceToDevice, st));
        off += pc;
      }
      FML_REQUIRE(ctx, off == o.cols, where + " (concat): part widths do not add up to cols");
      return FML_OK;
    }
    case FML_OP_SOFTMAX_MATRIX:
      FML_REQUIRE(ctx, o.in[0], where + " (softmax_matrix): missing input");
      return fml_softmax_rows_fwd(ctx, o.in[0], o.out, o.rows, o.cols, 1.f, o.iparam);
    case FML_OP_LAYER_NORM:
      FML_REQUIRE(ctx, o.in[0] && o.in[1] && o.in[2] && o.aux[0] && o.aux[1], where + " (layer_norm): missing input or aux buffer");
      return fml_layernorm_fwd(ctx, o.in[0], nullptr, o.in[1], o.in[2], o.out, o.aux[0], o.aux[1], o.rows, o.cols, o.s);
    case FML_OP_EMBEDDING_LOOKUP:
      FML_REQUIRE(ctx, o.in[0] && o.ids, where + " (embedding_lookup): missing table or ids");
      return fml_embedding_fwd(ctx, o.in[0], o.ids, nullptr, o.out, o.rows, o.cols, 0, o.inner);
    case FML_OP_MSE: {
      FML_REQUIRE(ctx, o.in[0] && o.in[1] && o.inner > 0, where + " (mse): missing input (inner = element count)");
      TP_TRY(fml_zero(ctx, o.out, 1));
      return fml_mse(ctx, o.in[0], o.in[1], nullptr, o.out, o.inner, 1.f);
    }
    case FML_OP_SUM: {
      FML_REQUIRE(ctx, o.in[0] && o.inner > 0, where + " (sum): missing input (inner = element count)");
      const int blocks = tp_blocks(ctx, o.inner);
      TP_TRY(fml_ensure_workspace(ctx, (size_t)blocks * sizeof(double)));
      sum_partial_kernel<<<blocks, TP_THREADS, 0, st>>>(o.in[0], reinterpret_cast<double*>(ctx->ws), o.inner);
      sum_final_kernel<<<1, TP_THREADS, 0, st>>>(reinterpret_cast<const double*>(ctx->ws), blocks, o.out);
      FML_LAUNCH_CHECK(ctx, "sum_kernel");
      return FML_OK;
    }
    case FML_OP_ATTENTION: {
      fml_attention_desc d;
      TP_TRY(attention_desc_of(ctx, o, where, &d));
      return fml_attention_fwd(ctx, &d);
    }
    case FML_OP_CONV2D: {
      const int pad = (int)o.s, H = o.rows + o.inner - 1 - 2 * pad, W = o.cols + o.iparam - 1 - 2 * pad;
      FML_REQUIRE(ctx, o.in[0] && o.in[1] && o.inner > 0 && o.iparam > 0 && pad >= 0 && H > 0 && W > 0, where + " (conv2d): bad input, kernel or padding");
      return fml_conv2d_fwd(ctx, o.in[0], o.in[1], nullptr, o.out, 1, H, W, 1, o.inner, o.iparam, pad);
    }
    case FML_OP_ADD_SCALAR_TO_MATRIX:
      FML_REQUIRE(ctx, o.in[0] && o.in[1], where + " (addScalarToMatrix): missing input");
      add_scalar_dev_kernel<<<tp_blocks(ctx, n), TP_THREADS, 0, st>>>(o.in[0], o.in[1], o.out, n);
      FML_LAUNCH_CHECK(ctx, "add_scalar_dev_kernel");
      return FML_OK;
    case FML_OP_SOFTMAX_XENT: {
      FML_REQUIRE(ctx, o.in[0] && o.ids && o.aux[0] && o.inner > 0, where + " (softmax_xent): missing logits, labels or aux[0]");
      TP_TRY(fml_zero(ctx, o.out, 1));
      return fml_softmax_xent(ctx, o.in[0], o.ids, o.aux[0], o.out, o.inner, o.iparam, o.s);
    }
    default:
      return fml_fail(ctx, FML_ERR_INVALID, where + ": unknown kind " + std::to_string(o.kind));
  }
}

}  // namespace

namespace {

// gin += g (add fan-in); no-op for a NULL target
int32_t acc_into(fml_ctx* ctx, float* gin, const float* g, long long n) {
  return gin ? fml_axpy(ctx, 1.f, g, gin, n) : FML_OK;
}

int32_t op_backward(fml_ctx* ctx, const fml_op& o, int idx) {
  const long long n = (long long)o.rows * o.cols;
  const std::string where = "fml_tape_run: op " + std::to_string(idx);
  FML_REQUIRE(ctx, o.gout, where + ": gout is NULL in the backward sweep");
  cudaStream_t st = ctx->stream;
  switch (o.kind) {
    case FML_OP_MATMUL:
      // dA += dC . B^T (tensor.dart:918-924), dB += A^T . dC (tensor.dart:935-941)
      if (o.gin[0]) TP_TRY(tp_gemm(ctx, o.gout, o.in[1], o.gin[0], o.rows, o.inner, o.cols, false, true, 1.f, o.precision));
      if (o.gin[1]) TP_TRY(tp_gemm(ctx, o.in[0], o.gout, o.gin[1], o.inner, o.cols, o.rows, true, false, 1.f, o.precision));
      return FML_OK;
    case FML_OP_DENSE: {
      const float* dz = o.gout;
      if (o.iparam != FML_ACT_NONE) {
        // dZ = dY * act'(.) and the bias gradient in one pass; dZ overwrites gout, which nothing reads afterwards
        const float* saved = o.iparam == FML_ACT_GELU ? o.aux[0] : o.out;
        TP_TRY(fml_act_bwd(ctx, o.iparam, saved, o.gout, o.gout, o.rows, o.cols, 0, o.gin[2]));
      } else if (o.gin[2]) {
        TP_TRY(fml_col_sum(ctx, dz, o.gin[2], o.rows, o.cols, 1));
      }
      if (o.gin[0]) TP_TRY(tp_gemm(ctx, dz, o.in[1], o.gin[0], o.rows, o.inner, o.cols, false, true, 1.f, o.precision));
      if (o.gin[1]) TP_TRY(tp_gemm(ctx, o.in[0], dz, o.gin[1], o.inner, o.cols, o.rows, true, false, 1.f, o.precision));
      return FML_OK;
    }
    case FML_OP_MATVECMUL: {
      if (!o.gin[0] && !o.gin[1]) return FML_OK;
      const int rows = o.cols, cols = o.inner;  // the matrix is cols(out) x inner
      const int cb = (cols + TP_THREADS - 1) / TP_THREADS;
      int rb = std::max(1, std::min((rows + 15) / 16, (ctx->sm_count * 8 + cb - 1) / cb));
      const int rpb = (rows + rb - 1) / rb;
      rb = (rows + rpb - 1) / rpb;
      gemv_bwd_kernel<<<dim3(cb, rb), TP_THREADS, 0, st>>>(o.in[0], o.in[1], o.gout, o.gin[0], o.gin[1], rows, cols, rpb);
      FML_LAUNCH_CHECK(ctx, "gemv_bwd_kernel");
      return FML_OK;
    }
    case FML_OP_ADD_MATRIX_AND_VECTOR:
      TP_TRY(acc_into(ctx, o.gin[0], o.gout, n));
      if (o.gin[1]) TP_TRY(fml_col_sum(ctx, o.gout, o.gin[1], o.rows, o.cols, 1));
      return FML_OK;
    case FML_OP_ADD:
      TP_TRY(acc_into(ctx, o.gin[0], o.gout, n));
      return acc_into(ctx, o.gin[1], o.gout, n);
    case FML_OP_MULTIPLY:
      if (o.gin[0]) mul_acc_kernel<<<tp_blocks(ctx, n), TP_THREADS, 0, st>>>(o.gout, o.in[1], o.gin[0], n);
      if (o.gin[1]) mul_acc_kernel<<<tp_blocks(ctx, n), TP_THREADS, 0, st>>>(o.gout, o.in[0], o.gin[1], n);
      FML_LAUNCH_CHECK(ctx, "mul_acc_kernel");
      return FML_OK;
    case FML_OP_RELU: case FML_OP_GELU:   // gate on the INPUT (tensor.dart:1030)
      return o.gin[0] ? fml_act_bwd(ctx, act_of_kind(o.kind), o.in[0], o.gout, o.gin[0], o.rows, o.cols, 1, nullptr) : FML_OK;
    case FML_OP_SIGMOID: case FML_OP_TANH:  // derivative from the OUTPUT (tensor.dart:552, 598)
      return o.gin[0] ? fml_act_bwd(ctx, act_of_kind(o.kind), o.out, o.gout, o.gin[0], o.rows, o.cols, 1, nullptr) : FML_OK;
    case FML_OP_LEAKY_RELU: case FML_OP_ELU: case FML_OP_SWISH: case FML_OP_MISH:
      return o.gin[0] ? fml_act2_bwd(ctx, act2_of_kind(o.kind), o.s, o.in[0], o.gout, o.gin[0], n, 1) : FML_OK;
    case FML_OP_SCALE_MATRIX:
      return o.gin[0] ? fml_axpy(ctx, o.s, o.gout, o.gin[0], n) : FML_OK;
    case FML_OP_TRANSPOSE: {
      if (!o.gin[0]) return FML_OK;
      dim3 grid((unsigned)((o.cols + 31) / 32), (unsigned)((o.rows + 31) / 32));
      FML_REQUIRE(ctx, grid.y <= 65535, where + " (transpose): too many rows");
      transpose_acc_kernel<<<grid, TP_THREADS, 0, st>>>(o.gout, o.gin[0], o.rows, o.cols);
      FML_LAUNCH_CHECK(ctx, "transpose_acc_kernel");
      return FML_OK;
    }
    case FML_OP_CONCAT: {
      if (!o.gparts) return FML_OK;
      int off = 0;
      for (int p = 0; p < o.n_parts; p++) {
        const int pc = o.part_cols[p];
        if (o.gparts[p])
          split_add_kernel<<<tp_blocks(ctx, (long long)o.rows * pc), TP_THREADS, 0, st>>>(o.gparts[p], o.gout, o.rows, pc, o.cols, off);
        off += pc;
      }
      FML_LAUNCH_CHECK(ctx, "split_add_kernel");
      return FML_OK;
    }
    case FML_OP_SOFTMAX_MATRIX:
      return o.gin[0] ? fml_softmax_rows_bwd(ctx, o.out, o.gout, o.gin[0], o.rows, o.cols, 1.f, 1) : FML_OK;
    case FML_OP_LAYER_NORM:
      return fml_layernorm_bwd(ctx, o.gout, o.in[1], o.aux[0], o.aux[1], o.gin[0], o.gin[1], o.gin[2], o.rows, o.cols, 1);
    case FML_OP_EMBEDDING_LOOKUP:
      return o.gin[0] ? fml_embedding_bwd(ctx, o.gout, o.ids, o.gin[0], o.rows, o.cols, o.inner) : FML_OK;
    case FML_OP_MSE:
      if (o.gin[0]) {
        mse_bwd_kernel<<<tp_blocks(ctx, o.inner), TP_THREADS, 0, st>>>(o.in[0], o.in[1], o.gout, o.gin[0], 2.f / (float)o.inner, o.inner);
        FML_LAUNCH_CHECK(ctx, "mse_bwd_kernel");
      }
      return FML_OK;
    case FML_OP_SUM:
      if (o.gin[0]) {
        broadcast_add_dev_kernel<<<tp_blocks(ctx, o.inner), TP_THREADS, 0, st>>>(o.gin[0], o.gout, o.inner);
        FML_LAUNCH_CHECK(ctx, "broadcast_add_dev_kernel");
      }
      return FML_OK;
    case FML_OP_ATTENTION: {
      if (!o.gin[0] && !o.gin[1] && !o.gin[2]) return FML_OK;
      FML_REQUIRE(ctx, o.gin[0] && o.gin[1] && o.gin[2], where + " (attention): dQ, dK and dV are produced together; give all three or none");
      fml_attention_desc d;
      TP_TRY(attention_desc_of(ctx, o, where, &d));
      return fml_attention_bwd(ctx, &d, o.gout, o.cols, o.gin[0], o.gin[1], o.gin[2], o.cols, 1, o.aux[1]);
    }
    case FML_OP_CONV2D: {
      const int pad = (int)o.s, H = o.rows + o.inner - 1 - 2 * pad, W = o.cols + o.iparam - 1 - 2 * pad;
      if (!o.gin[0] && !o.gin[1]) return FML_OK;
      return fml_conv2d_bwd(ctx, o.in[0], o.in[1], o.gout, o.gin[0], o.gin[1], nullptr, 1, H, W, 1, o.inner, o.iparam, pad);
    }
    case FML_OP_ADD_SCALAR_TO_MATRIX:
      TP_TRY(acc_into(ctx, o.gin[0], o.gout, n));
      if (o.gin[1]) {  // s.grad += sum of out.grad (tensor.dart:729)
        const int blocks = tp_blocks(ctx, n);
        TP_TRY(fml_ensure_workspace(ctx, (size_t)(blocks + 1) * sizeof(double)));
        double* part = reinterpret_cast<double*>(ctx->ws);
        sum_partial_kernel<<<blocks, TP_THREADS, 0, st>>>(o.gout, part, n);
        sum_final_kernel<<<1, TP_THREADS, 0, st>>>(part, blocks, reinterpret_cast<float*>(part + blocks));
        add_one_dev_kernel<<<1, 1, 0, st>>>(o.gin[1], reinterpret_cast<const float*>(part + blocks));
        FML_LAUNCH_CHECK(ctx, "add_scalar backward");
      }
      return FML_OK;
    case FML_OP_SOFTMAX_XENT:
      if (o.gin[0]) {
        const long long m = (long long)o.inner * o.iparam;
        scaled_add_dev_kernel<<<tp_blocks(ctx, m), TP_THREADS, 0, st>>>(o.gin[0], o.aux[0], o.gout, 1.f, m);
        FML_LAUNCH_CHECK(ctx, "scaled_add_dev_kernel");
      }
      return FML_OK;
    default:
      return fml_fail(ctx, FML_ERR_INVALID, where + ": unknown kind " + std::to_string(o.kind));
  }
}

struct KindName { const char* name; int kind; };
const KindName KIND_NAMES[] = {
    {"matMul", FML_OP_MATMUL}, {"matVecMul", FML_OP_MATVECMUL}, {"addMatrixAndVector", FML_OP_ADD_MATRIX_AND_VECTOR},
    {"add_matrix", FML_OP_ADD}, {"add_vector", FML_OP_ADD}, {"add_3d", FML_OP_ADD},
    {"multiply_matrix", FML_OP_MULTIPLY}, {"multiply_vector", FML_OP_MULTIPLY}, {"multiply_3d", FML_OP_MULTIPLY},
    {"relu_matrix", FML_OP_RELU}, {"relu_vector", FML_OP_RELU}, {"sigmoid_matrix", FML_OP_SIGMOID},
    {"sigmoid_vector", FML_OP_SIGMOID}, {"tanh_matrix", FML_OP_TANH}, {"tanh_vector", FML_OP_TANH}, {"gelu", FML_OP_GELU},
    {"leaky_relu", FML_OP_LEAKY_RELU}, {"elu", FML_OP_ELU}, {"elu_matrix", FML_OP_ELU}, {"swish", FML_OP_SWISH},
    {"mish", FML_OP_MISH}, {"scale_matrix", FML_OP_SCALE_MATRIX}, {"transpose", FML_OP_TRANSPOSE},
    {"concat_matrix_col", FML_OP_CONCAT}, {"concat_vector", FML_OP_CONCAT}, {"softmax_matrix", FML_OP_SOFTMAX_MATRIX},
    {"softmax", FML_OP_SOFTMAX_MATRIX}, {"layer_norm", FML_OP_LAYER_NORM}, {"layer_norm_vector", FML_OP_LAYER_NORM},
    {"embedding_lookup", FML_OP_EMBEDDING_LOOKUP}, {"mse_matrix", FML_OP_MSE}, {"mse_vector", FML_OP_MSE},
    {"attention", FML_OP_ATTENTION}, {"conv2d", FML_OP_CONV2D}, {"addScalarToMatrix", FML_OP_ADD_SCALAR_TO_MATRIX}, {"sum_matrix", FML_OP_SUM}, {"sum_vector", FML_OP_SUM}, {"softmax_xent", FML_OP_SOFTMAX_XENT}, {"dense", FML_OP_DENSE},
    {"dense_matrix", FML_OP_DENSE}};

}  // namespace

extern "C" {

int32_t fml_tape_kind(const char* op_name) {
  if (!op_name) return 0;
  for (const KindName& k : KIND_NAMES)
    if (std::strcmp(k.name, op_name) == 0) return k.kind;
  return 0;
}

int32_t fml_tape_run(fml_ctx* ctx, const fml_op* ops, int32_t n_ops, int32_t direction) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, ctx && n_ops >= 0 && (ops || n_ops == 0), "fml_tape_run: bad arguments");
  FML_REQUIRE(ctx, direction >= FML_TAPE_FORWARD && direction <= FML_TAPE_BACKWARD_NOSEED, "fml_tape_run: unknown direction");
  if (n_ops == 0) return FML_OK;
  if (direction == FML_TAPE_FORWARD) {
    for (int i = 0; i < n_ops; i++) TP_TRY(op_forward(ctx, ops[i], i));
    return FML_OK;
  }
  if (direction == FML_TAPE_BACKWARD) {
    const fml_op& last = ops[n_ops - 1];
    FML_REQUIRE(ctx, last.gout && last.rows > 0 && last.cols > 0, "fml_tape_run: the last op has no gout to seed");
    TP_TRY(fml_fill(ctx, last.gout, (long long)last.rows * last.cols, 1.f));  // this.grad = 1.0, tensor.dart:70
  }
  for (int i = n_ops - 1; i >= 0; i--) TP_TRY(op_backward(ctx, ops[i], i));
  return FML_OK;
}

}  // extern "C"
