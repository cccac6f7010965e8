// Memory-bound elementwise kernels: activations and their gradients, adds, optimizer updates,
// embedding gather / scatter-add, column sums, transpose.  All of them stream with 128-bit
// loads and stores when the pointers allow it (scalar tail otherwise) on a grid of a few CTAs
// per SM walking the array with a grid stride.
#include <algorithm>

#include "common.cuh"

namespace {

constexpr int EW_THREADS = 256;

inline int ew_blocks(fml_ctx* ctx, long long work_items) {
  long long b = (work_items + EW_THREADS - 1) / EW_THREADS;
  return (int)std::max<long long>(1, std::min<long long>(b, (long long)ctx->sm_count * 8));
}
inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

#define EW_LOOP(i, n) \
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (n); i += (long long)gridDim.x * blockDim.x)

// ------------------------------------------------------------------ activations
template <bool VEC>
__global__ void act_fwd_kernel(int act, const float* __restrict__ x, float* __restrict__ y, long long n) {
  if (VEC) {
    EW_LOOP(i, n >> 2) {
      float4 v = reinterpret_cast<const float4*>(x)[i];
      v.x = fml_act_apply(act, v.x); v.y = fml_act_apply(act, v.y);
      v.z = fml_act_apply(act, v.z); v.w = fml_act_apply(act, v.w);
      reinterpret_cast<float4*>(y)[i] = v;
    }
  } else {
    EW_LOOP(i, n) y[i] = fml_act_apply(act, x[i]);
  }
}

template <bool VEC>
__global__ void act_bwd_kernel(int act, const float* __restrict__ s, const float* __restrict__ dy, float* dx,
                               long long n, int accumulate) {
  if (VEC) {
    EW_LOOP(i, n >> 2) {
      float4 sv = reinterpret_cast<const float4*>(s)[i];
      float4 g = reinterpret_cast<const float4*>(dy)[i];
      float4 o;
      o.x = g.x * fml_act_grad(act, sv.x); o.y = g.y * fml_act_grad(act, sv.y);
      o.z = g.z * fml_act_grad(act, sv.z); o.w = g.w * fml_act_grad(act, sv.w);
      if (accumulate) {
        float4 old = reinterpret_cast<float4*>(dx)[i];
        o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
      }
      reinterpret_cast<float4*>(dx)[i] = o;
    }
  } else {
    EW_LOOP(i, n) {
      float o = dy[i] * fml_act_grad(act, s[i]);
      dx[i] = accumulate ? dx[i] + o : o;
    }
  }
}

// dx = dy * act'(saved) and db[c] += column sums of dx in ONE pass over the data: a block owns 128
// columns (one float4 per lane) and a slab of rows; each warp walks its rows with 512-byte
// coalesced loads, keeps four column partials per lane in registers, and the block issues one
// atomic per column at the end.
__global__ void __launch_bounds__(256) act_bwd_colsum_kernel(int act, const float* __restrict__ s,
                                                             const float* __restrict__ dy, float* __restrict__ dx,
                                                             float* db, long long rows, long long cols,
                                                             long long rows_per_block) {
  __shared__ float red[8][128];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long c = blockIdx.x * 128ll + lane * 4;
  const long long r0 = blockIdx.y * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c < cols) {
    for (long long r = r0 + warp; r < r1; r += 8) {
      const long long o = r * cols + c;
      const float4 sv = *reinterpret_cast<const float4*>(s + o);
      const float4 g = *reinterpret_cast<const float4*>(dy + o);
      float4 d;
      d.x = g.x * fml_act_grad(act, sv.x); d.y = g.y * fml_act_grad(act, sv.y);
      d.z = g.z * fml_act_grad(act, sv.z); d.w = g.w * fml_act_grad(act, sv.w);
      *reinterpret_cast<float4*>(dx + o) = d;
      acc.x += d.x; acc.y += d.y; acc.z += d.z; acc.w += d.w;
    }
  }
  red[warp][lane * 4 + 0] = acc.x; red[warp][lane * 4 + 1] = acc.y;
  red[warp][lane * 4 + 2] = acc.z; red[warp][lane * 4 + 3] = acc.w;
  __syncthreads();
  if (threadIdx.x < 128) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) t += red[w][threadIdx.x];
    const long long col = blockIdx.x * 128ll + threadIdx.x;
    if (col < cols) atomicAdd(db + col, t);
  }
}

// ------------------------------------------------------------------ binary ops
// mode 0: y = a + b; 1: y = a * b; 2: y = y + s * a (b unused)
template <bool VEC>
__global__ void binary_kernel(int mode, float s, const float* a, const float* b, float* y, long long n) {
  if (VEC) {
    EW_LOOP(i, n >> 2) {
      float4 av = reinterpret_cast<const float4*>(a)[i];
      float4 o;
      if (mode == 2) {
        float4 yv = reinterpret_cast<float4*>(y)[i];
        o.x = yv.x + s * av.x; o.y = yv.y + s * av.y; o.z = yv.z + s * av.z; o.w = yv.w + s * av.w;
      } else {
        float4 bv = reinterpret_cast<const float4*>(b)[i];
        if (mode == 0) { o.x = av.x + bv.x; o.y = av.y + bv.y; o.z = av.z + bv.z; o.w = av.w + bv.w; }
        else { o.x = av.x * bv.x; o.y = av.y * bv.y; o.z = av.z * bv.z; o.w = av.w * bv.w; }
      }
      reinterpret_cast<float4*>(y)[i] = o;
    }
  } else {
    EW_LOOP(i, n) {
      if (mode == 2) y[i] = y[i] + s * a[i];
      else if (mode == 0) y[i] = a[i] + b[i];
      else y[i] = a[i] * b[i];
    }
  }
}

__global__ void fill_kernel(float* __restrict__ p, long long n, float value) {
  EW_LOOP(i, n) p[i] = value;
}

__global__ void add_bias_kernel(const float* __restrict__ x, const float* __restrict__ b, float* __restrict__ y,
                                long long rows, long long cols) {
  EW_LOOP(i, rows * cols) y[i] = x[i] + b[i % cols];
}

// db[c] (+)= sum over rows of dy[r][c]; block (32 x 8) covers 32 columns and a slab of rows
__global__ void col_sum_kernel(const float* __restrict__ dy, float* db, long long rows, long long cols,
                               long long rows_per_block) {
  __shared__ float red[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long long c = blockIdx.x * 32ll + tx;
  const long long r0 = blockIdx.y * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  float acc = 0.f;
  if (c < cols)
    for (long long r = r0 + ty; r < r1; r += 8) acc += dy[r * cols + c];
  red[ty][tx] = acc;
  __syncthreads();
  if (ty == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; k++) t += red[k][tx];
    atomicAdd(db + c, t);
  }
}

__global__ void transpose_kernel(const float* __restrict__ in, float* __restrict__ out, long long rows, long long cols) {
  __shared__ float tile[32][33];
  const long long c0 = blockIdx.x * 32ll, r0 = blockIdx.y * 32ll;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int k = ty; k < 32; k += 8)
    if (r0 + k < rows && c0 + tx < cols) tile[k][tx] = in[(r0 + k) * cols + c0 + tx];
  __syncthreads();
  for (int k = ty; k < 32; k += 8)
    if (c0 + k < cols && r0 + tx < rows) out[(c0 + k) * rows + r0 + tx] = tile[tx][k];
}

// ------------------------------------------------------------------ optimizers
template <bool VEC>
__global__ void sgd_kernel(float* w, const float* __restrict__ g, long long n, float lr, float gs) {
  if (VEC) {
    EW_LOOP(i, n >> 2) {
      float4 wv = reinterpret_cast<float4*>(w)[i];
      float4 gv = reinterpret_cast<const float4*>(g)[i];
      wv.x -= lr * (gs * gv.x); wv.y -= lr * (gs * gv.y); wv.z -= lr * (gs * gv.z); wv.w -= lr * (gs * gv.w);
      reinterpret_cast<float4*>(w)[i] = wv;
    }
  } else {
    EW_LOOP(i, n) w[i] -= lr * (gs * g[i]);
  }
}

// bias corrections 1 - beta^t are computed once on the host in double (the reference evaluates
// pow(beta, t) per element, adam.dart:57-58; the value is the same)
struct AdamK { float lr, b1, b2, omb1, omb2, eps, c1, c2, gs; };
__device__ __forceinline__ void adam1(float& w, float g, float& m, float& v, const AdamK& k) {
  const float lr = k.lr, b1 = k.b1, b2 = k.b2, eps = k.eps, c1 = k.c1, c2 = k.c2;
  m = b1 * m + k.omb1 * g;
  v = b2 * v + k.omb2 * (g * g);
  const float mh = m / c1, vh = v / c2;
  w -= lr * mh / (sqrtf(vh) + eps);
}
// ZERO: the gradient is cleared as it is consumed (Optimizer.zeroGrad, optimizers.dart:62-66, folded into the
// update: one pass over the gradient instead of a read here and a memset later).
template <bool VEC, bool ZERO>
__global__ void adam_kernel(float* __restrict__ w, float* __restrict__ g, float* __restrict__ m, float* __restrict__ v, long long n,
                            const AdamK k) {
  const float gs = k.gs;
  if (VEC) {
    // All four loads first, the stores (the cleared gradient among them) last: with the gradient cleared between the
    // loads, and pointers that may alias, the compiler kept the loads of m and v behind that store and the kernel ran at
    // 1.6 TB/s instead of 6.2 (measured on the 33 M-parameter slice of the language-model step).
    EW_LOOP(i, n >> 2) {
      float4 wv = reinterpret_cast<const float4*>(w)[i];
      const float4 gv = reinterpret_cast<const float4*>(g)[i];
      float4 mv = reinterpret_cast<const float4*>(m)[i];
      float4 vv = reinterpret_cast<const float4*>(v)[i];
      adam1(wv.x, gs * gv.x, mv.x, vv.x, k);
      adam1(wv.y, gs * gv.y, mv.y, vv.y, k);
      adam1(wv.z, gs * gv.z, mv.z, vv.z, k);
      adam1(wv.w, gs * gv.w, mv.w, vv.w, k);
      reinterpret_cast<float4*>(w)[i] = wv;
      reinterpret_cast<float4*>(m)[i] = mv;
      reinterpret_cast<float4*>(v)[i] = vv;
      if (ZERO) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  } else {
    EW_LOOP(i, n) {
      const float gi = g[i];
      adam1(w[i], gs * gi, m[i], v[i], k);
      if (ZERO) g[i] = 0.f;
    }
  }
}

struct OptK { float lr, h1, h2, h3, h4, omh1, omh2, c1, c2; int kind; };
__global__ void optimizer_kernel(float* w, const float* __restrict__ g, float* s1, float* s2, float* s3, long long n, const OptK k) {
  EW_LOOP(i, n) {
    const float gi = g[i];
    float wi = w[i];
    switch (k.kind) {
      case FML_OPT_MOMENTUM: { const float v = k.h1 * s1[i] + k.lr * gi; s1[i] = v; wi -= v; break; }
      case FML_OPT_NAG: { const float v = k.h1 * s1[i] + gi; s1[i] = v; wi -= k.lr * (gi + k.h1 * v); break; }
      case FML_OPT_RMSPROP: { const float s = k.h1 * s1[i] + k.omh1 * (gi * gi); s1[i] = s; wi -= k.lr * gi / (sqrtf(s) + k.h2); break; }
      case FML_OPT_ADAGRAD: { const float s = s1[i] + gi * gi; s1[i] = s; wi -= k.lr * gi / (sqrtf(s) + k.h2); break; }
      case FML_OPT_ADAMW: {
        const float m = k.h1 * s1[i] + k.omh1 * gi, v = k.h2 * s2[i] + k.omh2 * (gi * gi);
        s1[i] = m; s2[i] = v;
        wi -= k.lr * (m / k.c1) / (sqrtf(v / k.c2) + k.h3);
        wi -= k.lr * k.h4 * wi;
        break;
      }
      case FML_OPT_AMSGRAD: {
        const float m = k.h1 * s1[i] + k.omh1 * gi, v = k.h2 * s2[i] + k.omh2 * (gi * gi);
        const float vh = fmaxf(s3[i], v);
        s1[i] = m; s2[i] = v; s3[i] = vh;
        wi -= k.lr * (m / k.c1) / (sqrtf(vh) + k.h3);
        break;
      }
      default: break;
    }
    w[i] = wi;
  }
}

// tanh(log(1 + e^x)) = ((1+e^x)^2 - 1) / ((1+e^x)^2 + 1) = n / (n + 2) with n = e^x (e^x + 2): no cancellation for
// negative x, and 1 to float precision once e^x > 2^12.
__device__ __forceinline__ float mish_tanh_softplus(float v) {
  if (v > 20.f) return 1.f;
  const float e = expf(v), n = e * (e + 2.f);
  return n / (n + 2.f);
}
__device__ __forceinline__ float act2_apply(int kind, float alpha, float v) {
  switch (kind) {
    case FML_ACT2_LEAKY_RELU: return v > 0.f ? v : alpha * v;
    case FML_ACT2_ELU: return v > 0.f ? v : alpha * (expf(v) - 1.f);
    case FML_ACT2_SWISH: return v * (1.f / (1.f + expf(-v)));
    case FML_ACT2_MISH: return v * mish_tanh_softplus(v);
    default: return v;
  }
}
__device__ __forceinline__ float act2_grad(int kind, float alpha, float v) {
  switch (kind) {
    case FML_ACT2_LEAKY_RELU: return v > 0.f ? 1.f : alpha;
    case FML_ACT2_ELU: return v > 0.f ? 1.f : alpha * (expf(v) - 1.f) + alpha;
    case FML_ACT2_SWISH: { const float sg = 1.f / (1.f + expf(-v)); return sg * (1.f + v * (1.f - sg)); }
    case FML_ACT2_MISH: {
      const float th = mish_tanh_softplus(v), sg = 1.f / (1.f + expf(-v));
      return th + v * (1.f - th * th) * sg;
    }
    default: return 1.f;
  }
}
__global__ void act2_fwd_kernel(int kind, float alpha, const float* __restrict__ x, float* __restrict__ y, long long n) {
  EW_LOOP(i, n) y[i] = act2_apply(kind, alpha, x[i]);
}
__global__ void act2_bwd_kernel(int kind, float alpha, const float* __restrict__ x, const float* __restrict__ dy, float* dx,
                                long long n, int accumulate) {
  EW_LOOP(i, n) {
    const float o = dy[i] * act2_grad(kind, alpha, x[i]);
    dx[i] = accumulate ? dx[i] + o : o;
  }
}

// ------------------------------------------------------------------ embedding
// A token id outside [0, vocab) reads nothing (its row comes out as the positional part only) and is reported
// through the status block; the reference would throw a RangeError at embeddingLayer.dart:53.
__global__ void embedding_fwd_kernel(const float* __restrict__ table, const int* __restrict__ ids,
                                     const float* __restrict__ pe, float* __restrict__ out, long long n, int dim,
                                     int period, int vocab, int* status) {
  const int d4 = dim >> 2;
  EW_LOOP(i, n * d4) {
    const long long r = i / d4;
    const int c = (int)(i % d4);
    const int id = ids[r];
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if ((unsigned)id < (unsigned)vocab) v = reinterpret_cast<const float4*>(table + (long long)id * dim)[c];
    else if (c == 0) fml_flag_bad_index(status, FML_BAD_INDEX_EMBEDDING_FWD);
    if (pe) {
      float4 q = reinterpret_cast<const float4*>(pe + (r % period) * dim)[c];
      v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
    }
    reinterpret_cast<float4*>(out + r * dim)[c] = v;
  }
}
__global__ void embedding_fwd_scalar_kernel(const float* __restrict__ table, const int* __restrict__ ids,
                                            const float* __restrict__ pe, float* __restrict__ out, long long n, int dim,
                                            int period, int vocab, int* status) {
  EW_LOOP(i, n * dim) {
    const long long r = i / dim;
    const int c = (int)(i % dim);
    const int id = ids[r];
    float v = 0.f;
    if ((unsigned)id < (unsigned)vocab) v = table[(long long)id * dim + c];
    else if (c == 0) fml_flag_bad_index(status, FML_BAD_INDEX_EMBEDDING_FWD);
    if (pe) v += pe[(r % period) * dim + c];
    out[i] = v;
  }
}
__global__ void embedding_bwd_kernel(const float* __restrict__ dout, const int* __restrict__ ids, float* dtable,
                                     long long n, int dim, int vocab, int* status) {
  EW_LOOP(i, n * dim) {
    const long long r = i / dim;
    const int c = (int)(i % dim);
    const int id = ids[r];
    if ((unsigned)id < (unsigned)vocab) atomicAdd(dtable + (long long)id * dim + c, dout[i]);
    else if (c == 0) fml_flag_bad_index(status, FML_BAD_INDEX_EMBEDDING_BWD);
  }
}
__global__ void positional_kernel(float* pe, int max_len, int d_model) {
  EW_LOOP(i, (long long)max_len * d_model) {
    const int pos = (int)(i / d_model), c = (int)(i % d_model);
    // evaluated in double: this table is built once and the reference builds it in float64
    const double angle = (double)pos / pow(10000.0, (2.0 * c) / (double)d_model);
    pe[i] = (float)((c % 2 == 0) ? sin(angle) : cos(angle));
  }
}

template <class K, class... Args>
int32_t launch_vec(fml_ctx* ctx, const char* name, bool vec, long long n, K kvec, K kscalar, Args... args) {
  if (n <= 0) return FML_OK;
  if (vec) kvec<<<ew_blocks(ctx, n >> 2), EW_THREADS, 0, ctx->stream>>>(args...);
  else kscalar<<<ew_blocks(ctx, n), EW_THREADS, 0, ctx->stream>>>(args...);
  FML_LAUNCH_CHECK(ctx, name);
  return FML_OK;
}

}  // namespace

extern "C" {

int32_t fml_fill(fml_ctx* ctx, float* p, int64_t n, float value) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, p && n >= 0, "fml_fill: bad arguments");
  if (n == 0) return FML_OK;
  fill_kernel<<<ew_blocks(ctx, n), EW_THREADS, 0, ctx->stream>>>(p, n, value);
  FML_LAUNCH_CHECK(ctx, "fill_kernel");
  return FML_OK;
}

int32_t fml_act_fwd(fml_ctx* ctx, int32_t act, const float* x, float* y, int64_t n) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, x && y && n >= 0, "fml_act_fwd: bad arguments");
  const bool vec = (n % 4 == 0) && al16(x) && al16(y);
  return launch_vec(ctx, "act_fwd_kernel", vec, n, act_fwd_kernel<true>, act_fwd_kernel<false>, act, x, y, (long long)n);
}

int32_t fml_col_sum(fml_ctx* ctx, const float* dy, float* db, int64_t rows, int64_t cols, int32_t accumulate) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, dy && db && rows > 0 && cols > 0, "fml_col_sum: bad arguments");
  if (!accumulate) FML_CUDA(ctx, cudaMemsetAsync(db, 0, (size_t)cols * 4, ctx->stream));
  const long long cb = (cols + 31) / 32;
  long long rb = std::max<long long>(1, std::min<long long>((rows + 63) / 64, ((long long)ctx->sm_count * 8 + cb - 1) / cb));
  const long long rows_per_block = (rows + rb - 1) / rb;
  rb = (rows + rows_per_block - 1) / rows_per_block;
  col_sum_kernel<<<dim3((unsigned)cb, (unsigned)rb), 256, 0, ctx->stream>>>(dy, db, rows, cols, rows_per_block);
  FML_LAUNCH_CHECK(ctx, "col_sum_kernel");
  return FML_OK;
}

int32_t fml_act_bwd(fml_ctx* ctx, int32_t act, const float* saved, const float* dy, float* dx, int64_t rows,
                    int64_t cols, int32_t accumulate, float* dbias) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, dy && dx && rows > 0 && cols > 0, "fml_act_bwd: bad arguments");
  FML_REQUIRE(ctx, act == FML_ACT_NONE || saved, "fml_act_bwd: saved tensor required");
  const long long n = rows * cols;
  if (act == FML_ACT_NONE) saved = dy;
  if (dbias && !accumulate && cols % 4 == 0 && al16(saved) && al16(dy) && al16(dx)) {
    const long long cb = (cols + 127) / 128;
    long long rb = std::max<long long>(1, std::min<long long>((rows + 31) / 32, ((long long)ctx->sm_count * 8 + cb - 1) / cb));
    const long long rows_per_block = (rows + rb - 1) / rb;
    rb = (rows + rows_per_block - 1) / rows_per_block;
    FML_REQUIRE(ctx, rb <= 65535, "fml_act_bwd: too many row slabs");
    act_bwd_colsum_kernel<<<dim3((unsigned)cb, (unsigned)rb), 256, 0, ctx->stream>>>(act, saved, dy, dx, dbias, rows, cols,
                                                                                    rows_per_block);
    FML_LAUNCH_CHECK(ctx, "act_bwd_colsum_kernel");
    return FML_OK;
  }
  const bool vec = (n % 4 == 0) && al16(saved) && al16(dy) && al16(dx);
  int32_t rc = launch_vec(ctx, "act_bwd_kernel", vec, n, act_bwd_kernel<true>, act_bwd_kernel<false>, act, saved, dy, dx, n,
                          accumulate);
  if (rc) return rc;
  if (dbias) {
    FML_REQUIRE(ctx, !accumulate, "fml_act_bwd: dbias needs the plain (non-accumulated) gradient in dx");
    return fml_col_sum(ctx, dx, dbias, rows, cols, 1);
  }
  return FML_OK;
}

static int32_t binary(fml_ctx* ctx, int mode, float s, const float* a, const float* b, float* y, int64_t n) {
  const bool vec = (n % 4 == 0) && al16(a) && al16(y) && (mode == 2 || al16(b));
  return launch_vec(ctx, "binary_kernel", vec, n, binary_kernel<true>, binary_kernel<false>, mode, s, a, b, y, (long long)n);
}
int32_t fml_add(fml_ctx* ctx, const float* a, const float* b, float* y, int64_t n) {
  FML_ENTER(ctx); return binary(ctx, 0, 0.f, a, b, y, n); }
int32_t fml_mul(fml_ctx* ctx, const float* a, const float* b, float* y, int64_t n) {
  FML_ENTER(ctx); return binary(ctx, 1, 0.f, a, b, y, n); }
int32_t fml_axpy(fml_ctx* ctx, float s, const float* x, float* y, int64_t n) {
  FML_ENTER(ctx); return binary(ctx, 2, s, x, nullptr, y, n); }

int32_t fml_add_bias(fml_ctx* ctx, const float* x, const float* b, float* y, int64_t rows, int64_t cols) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, x && b && y && rows > 0 && cols > 0, "fml_add_bias: bad arguments");
  add_bias_kernel<<<ew_blocks(ctx, rows * cols), EW_THREADS, 0, ctx->stream>>>(x, b, y, rows, cols);
  FML_LAUNCH_CHECK(ctx, "add_bias_kernel");
  return FML_OK;
}

int32_t fml_transpose(fml_ctx* ctx, const float* in, float* out, int64_t rows, int64_t cols) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, in && out && rows > 0 && cols > 0, "fml_transpose: bad arguments");
  dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32));
  FML_REQUIRE(ctx, grid.y <= 65535, "fml_transpose: too many rows");
  transpose_kernel<<<grid, 256, 0, ctx->stream>>>(in, out, rows, cols);
  FML_LAUNCH_CHECK(ctx, "transpose_kernel");
  return FML_OK;
}

int32_t fml_sgd_step(fml_ctx* ctx, float* w, const float* g, int64_t n, double lr, double grad_scale) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, w && g && n >= 0, "fml_sgd_step: bad arguments");
  const bool vec = (n % 4 == 0) && al16(w) && al16(g);
  return launch_vec(ctx, "sgd_kernel", vec, n, sgd_kernel<true>, sgd_kernel<false>, w, g, (long long)n, (float)lr, (float)grad_scale);
}

int32_t fml_adam_step(fml_ctx* ctx, float* w, const float* g, float* m, float* v, int64_t n, double lr, double beta1,
                      double beta2, double eps, int32_t t, double grad_scale) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, w && g && m && v && n >= 0 && t >= 1, "fml_adam_step: bad arguments");
  AdamK k;
  k.lr = (float)lr; k.b1 = (float)beta1; k.b2 = (float)beta2; k.eps = (float)eps; k.gs = (float)grad_scale;
  k.omb1 = (float)(1.0 - beta1); k.omb2 = (float)(1.0 - beta2);
  k.c1 = (float)(1.0 - pow(beta1, (double)t)); k.c2 = (float)(1.0 - pow(beta2, (double)t));
  const bool vec = (n % 4 == 0) && al16(w) && al16(g) && al16(m) && al16(v);
  return launch_vec(ctx, "adam_kernel", vec, n, adam_kernel<true, false>, adam_kernel<false, false>, w, const_cast<float*>(g), m, v,
                    (long long)n, k);
}

int32_t fml_adam_step_on(fml_ctx* ctx, int32_t lane, float* w, float* g, float* m, float* v, int64_t n, double lr, double beta1,
                         double beta2, double eps, int32_t t, double grad_scale, int32_t zero_grad) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, w && g && m && v && n >= 0 && t >= 1, "fml_adam_step_on: bad arguments");
  cudaStream_t s;
  int32_t rc = fml_any_stream(ctx, lane, &s);
  if (rc) return rc;
  AdamK k;
  k.lr = (float)lr; k.b1 = (float)beta1; k.b2 = (float)beta2; k.eps = (float)eps; k.gs = (float)grad_scale;
  k.omb1 = (float)(1.0 - beta1); k.omb2 = (float)(1.0 - beta2);
  k.c1 = (float)(1.0 - pow(beta1, (double)t)); k.c2 = (float)(1.0 - pow(beta2, (double)t));
  if (n == 0) return FML_OK;
  const bool vec = (n % 4 == 0) && al16(w) && al16(g) && al16(m) && al16(v);
  const int blocks = ew_blocks(ctx, vec ? n >> 2 : n);
  if (vec && zero_grad) adam_kernel<true, true><<<blocks, EW_THREADS, 0, s>>>(w, g, m, v, (long long)n, k);
  else if (vec) adam_kernel<true, false><<<blocks, EW_THREADS, 0, s>>>(w, g, m, v, (long long)n, k);
  else if (zero_grad) adam_kernel<false, true><<<blocks, EW_THREADS, 0, s>>>(w, g, m, v, (long long)n, k);
  else adam_kernel<false, false><<<blocks, EW_THREADS, 0, s>>>(w, g, m, v, (long long)n, k);
  FML_LAUNCH_CHECK(ctx, "adam_kernel");
  return FML_OK;
}

int32_t fml_optimizer_step(fml_ctx* ctx, int32_t kind, float* w, const float* g, float* s1, float* s2, float* s3, int64_t n,
                           double lr, double h1, double h2, double h3, double h4, int32_t t) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, w && g && n >= 0, "fml_optimizer_step: bad arguments");
  const bool two = kind == FML_OPT_ADAMW || kind == FML_OPT_AMSGRAD;
  FML_REQUIRE(ctx, kind == FML_OPT_MOMENTUM || kind == FML_OPT_NAG || kind == FML_OPT_RMSPROP || kind == FML_OPT_ADAGRAD || two,
              "fml_optimizer_step: unknown optimizer");
  FML_REQUIRE(ctx, s1 && (!two || s2) && (kind != FML_OPT_AMSGRAD || s3), "fml_optimizer_step: missing state buffer");
  FML_REQUIRE(ctx, !two || t >= 1, "fml_optimizer_step: t must be >= 1");
  OptK k;
  k.kind = kind; k.lr = (float)lr; k.h1 = (float)h1; k.h2 = (float)h2; k.h3 = (float)h3; k.h4 = (float)h4;
  k.omh1 = (float)(1.0 - h1); k.omh2 = (float)(1.0 - h2);
  k.c1 = two ? (float)(1.0 - pow(h1, (double)t)) : 1.f;
  k.c2 = two ? (float)(1.0 - pow(h2, (double)t)) : 1.f;
  if (n == 0) return FML_OK;
  optimizer_kernel<<<ew_blocks(ctx, n), EW_THREADS, 0, ctx->stream>>>(w, g, s1, s2, s3, n, k);
  FML_LAUNCH_CHECK(ctx, "optimizer_kernel");
  return FML_OK;
}

int32_t fml_act2_fwd(fml_ctx* ctx, int32_t kind, float alpha, const float* x, float* y, int64_t n) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, x && y && n >= 0 && kind >= FML_ACT2_LEAKY_RELU && kind <= FML_ACT2_MISH, "fml_act2_fwd: bad arguments");
  if (n == 0) return FML_OK;
  act2_fwd_kernel<<<ew_blocks(ctx, n), EW_THREADS, 0, ctx->stream>>>(kind, alpha, x, y, n);
  FML_LAUNCH_CHECK(ctx, "act2_fwd_kernel");
  return FML_OK;
}
int32_t fml_act2_bwd(fml_ctx* ctx, int32_t kind, float alpha, const float* x, const float* dy, float* dx, int64_t n,
                     int32_t accumulate) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, x && dy && dx && n >= 0 && kind >= FML_ACT2_LEAKY_RELU && kind <= FML_ACT2_MISH, "fml_act2_bwd: bad arguments");
  if (n == 0) return FML_OK;
  act2_bwd_kernel<<<ew_blocks(ctx, n), EW_THREADS, 0, ctx->stream>>>(kind, alpha, x, dy, dx, n, accumulate);
  FML_LAUNCH_CHECK(ctx, "act2_bwd_kernel");
  return FML_OK;
}

int32_t fml_embedding_fwd(fml_ctx* ctx, const float* table, const int32_t* ids, const float* pe, float* out, int64_t n,
                          int32_t dim, int32_t pe_period, int32_t vocab) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, table && ids && out && n > 0 && dim > 0 && vocab > 0, "fml_embedding_fwd: bad arguments");
  FML_REQUIRE(ctx, !pe || pe_period > 0, "fml_embedding_fwd: pe_period must be positive");
  if (dim % 4 == 0 && al16(table) && al16(out) && (!pe || al16(pe)))
    embedding_fwd_kernel<<<ew_blocks(ctx, n * (dim / 4)), EW_THREADS, 0, ctx->stream>>>(table, ids, pe, out, n, dim, pe_period, vocab, ctx->d_status);
  else
    embedding_fwd_scalar_kernel<<<ew_blocks(ctx, n * dim), EW_THREADS, 0, ctx->stream>>>(table, ids, pe, out, n, dim, pe_period, vocab, ctx->d_status);
  FML_LAUNCH_CHECK(ctx, "embedding_fwd_kernel");
  return FML_OK;
}

int32_t fml_embedding_bwd(fml_ctx* ctx, const float* dout, const int32_t* ids, float* dtable, int64_t n, int32_t dim,
                          int32_t vocab) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, dout && ids && dtable && n > 0 && dim > 0 && vocab > 0, "fml_embedding_bwd: bad arguments");
  embedding_bwd_kernel<<<ew_blocks(ctx, n * dim), EW_THREADS, 0, ctx->stream>>>(dout, ids, dtable, n, dim, vocab, ctx->d_status);
  FML_LAUNCH_CHECK(ctx, "embedding_bwd_kernel");
  return FML_OK;
}

int32_t fml_positional_table(fml_ctx* ctx, float* pe, int32_t max_len, int32_t d_model) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, pe && max_len > 0 && d_model > 0, "fml_positional_table: bad arguments");
  positional_kernel<<<ew_blocks(ctx, (long long)max_len * d_model), EW_THREADS, 0, ctx->stream>>>(pe, max_len, d_model);
  FML_LAUNCH_CHECK(ctx, "positional_kernel");
  return FML_OK;
}

}  // extern "C"
