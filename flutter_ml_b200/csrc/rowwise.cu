// Row kernels: softmax (with the attention scale and an optional causal mask folded in),
// layer normalisation (with the residual add folded in), softmax cross-entropy and MSE.
//
// Rows up to 2048 floats wide whose length is a multiple of 4 run one warp per row: each lane
// keeps its slice of the row in registers (float4 at lane + 32*i, so every load instruction of
// the warp covers 512 contiguous bytes), reductions are warp shuffles, and the row is read from
// HBM exactly once.  Other shapes take a block-per-row kernel.
#include <algorithm>

#include "common.cuh"

namespace {

constexpr float NEG_INF = -INFINITY;
inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// block-wide reductions for 256 threads
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int k = 0; k < 8; k++) t += red[k];
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = NEG_INF;
#pragma unroll
  for (int k = 0; k < 8; k++) t = fmaxf(t, red[k]);
  return t;
}

// ------------------------------------------------------------------------- softmax
template <int NV>
__global__ void __launch_bounds__(256) softmax_fwd_warp(const float* __restrict__ x, float* __restrict__ y, long long rows,
                                                        int cols, float scale, int causal_period) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = warp0; r < rows; r += nwarps) {
    const int lim = causal_period > 0 ? min(cols, (int)(r % causal_period) + 1) : cols;
    const float4* xr = reinterpret_cast<const float4*>(x + r * cols);
    // work in base 2: exp(s*x - m) = 2^(s*log2e*x - m'), one multiply folded into the scale
    const float k = scale * 1.4426950408889634f;
    float v[NV * 4];
    float mx = NEG_INF;
#pragma unroll
    for (int i = 0; i < NV; i++) {
      const int c = (lane + 32 * i) * 4;
      float4 t = make_float4(NEG_INF, NEG_INF, NEG_INF, NEG_INF);
      if (c < lim) t = xr[lane + 32 * i];  // columns at or beyond lim are masked below
      v[4 * i + 0] = (c + 0 < lim) ? t.x * k : NEG_INF;
      v[4 * i + 1] = (c + 1 < lim) ? t.y * k : NEG_INF;
      v[4 * i + 2] = (c + 2 < lim) ? t.z * k : NEG_INF;
      v[4 * i + 3] = (c + 3 < lim) ? t.w * k : NEG_INF;
#pragma unroll
      for (int e = 0; e < 4; e++) mx = fmaxf(mx, v[4 * i + e]);
    }
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV * 4; i++) {
      v[i] = fml_exp2_ftz(v[i] - mx);  // 2^(-inf) = 0 for masked columns
      s += v[i];
    }
    const float inv = 1.f / warp_sum(s);
    float4* yr = reinterpret_cast<float4*>(y + r * cols);
#pragma unroll
    for (int i = 0; i < NV; i++) {
      const int c = (lane + 32 * i) * 4;
      if (c < cols) yr[lane + 32 * i] = make_float4(v[4 * i] * inv, v[4 * i + 1] * inv, v[4 * i + 2] * inv, v[4 * i + 3] * inv);
    }
  }
}

template <int NV, bool ACC>
__global__ void __launch_bounds__(256) softmax_bwd_warp(const float* __restrict__ y, const float* __restrict__ dy, float* dx,
                                                        long long rows, int cols, float scale) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = warp0; r < rows; r += nwarps) {
    const float4* yr = reinterpret_cast<const float4*>(y + r * cols);
    const float4* gr = reinterpret_cast<const float4*>(dy + r * cols);
    float4 yv[NV], gv[NV];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; i++) {
      yv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      gv[i] = yv[i];
      if ((lane + 32 * i) * 4 < cols) { yv[i] = yr[lane + 32 * i]; gv[i] = gr[lane + 32 * i]; }
      dot += yv[i].x * gv[i].x + yv[i].y * gv[i].y + yv[i].z * gv[i].z + yv[i].w * gv[i].w;
    }
    float4* xr = reinterpret_cast<float4*>(dx + r * cols);
    float4 old[ACC ? NV : 1];
    if (ACC) {  // requested together with y and dy, ahead of the reduction
#pragma unroll
      for (int i = 0; i < NV; i++) {
        old[ACC ? i : 0] = make_float4(0.f, 0.f, 0.f, 0.f);
        if ((lane + 32 * i) * 4 < cols) old[ACC ? i : 0] = xr[lane + 32 * i];
      }
    }
    dot = warp_sum(dot);
#pragma unroll
    for (int i = 0; i < NV; i++) {
      if ((lane + 32 * i) * 4 < cols) {
        float4 o = make_float4(scale * yv[i].x * (gv[i].x - dot), scale * yv[i].y * (gv[i].y - dot),
                               scale * yv[i].z * (gv[i].z - dot), scale * yv[i].w * (gv[i].w - dot));
        if (ACC) { o.x += old[ACC ? i : 0].x; o.y += old[ACC ? i : 0].y; o.z += old[ACC ? i : 0].z; o.w += old[ACC ? i : 0].w; }
        xr[lane + 32 * i] = o;
      }
    }
  }
}

__global__ void __launch_bounds__(256) softmax_fwd_block(const float* __restrict__ x, float* __restrict__ y, long long rows,
                                                         int cols, float scale, int causal_period) {
  __shared__ float red[8];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const int lim = causal_period > 0 ? min(cols, (int)(r % causal_period) + 1) : cols;
    const float* xr = x + r * cols;
    float mx = NEG_INF;
    for (int c = threadIdx.x; c < lim; c += 256) mx = fmaxf(mx, xr[c] * scale);
    mx = block_max(mx, red);
    float s = 0.f;
    for (int c = threadIdx.x; c < lim; c += 256) s += expf(xr[c] * scale - mx);
    s = block_sum(s, red);
    for (int c = threadIdx.x; c < cols; c += 256) y[r * cols + c] = c < lim ? expf(xr[c] * scale - mx) / s : 0.f;
  }
}
__global__ void __launch_bounds__(256) softmax_bwd_block(const float* __restrict__ y, const float* __restrict__ dy, float* dx,
                                                         long long rows, int cols, float scale, int accumulate) {
  __shared__ float red[8];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    float dot = 0.f;
    for (int c = threadIdx.x; c < cols; c += 256) dot += y[r * cols + c] * dy[r * cols + c];
    dot = block_sum(dot, red);
    for (int c = threadIdx.x; c < cols; c += 256) {
      float o = scale * y[r * cols + c] * (dy[r * cols + c] - dot);
      dx[r * cols + c] = accumulate ? dx[r * cols + c] + o : o;
    }
  }
}

// ----------------------------------------------------------------------- layer norm
// RES is a template parameter on purpose: with a run-time `if (res)` around the second load the compiler keeps
// every load behind its branch and the warp waits out one memory round trip per float4 (0.78 of the copy
// bandwidth on 262144 x 1024); with all loads of a row issued back to back the kernel runs at 0.97.
template <int NV, bool RES>
__global__ void __launch_bounds__(256) layernorm_fwd_warp(const float* __restrict__ x, const float* __restrict__ res,
                                                          const float* __restrict__ gamma, const float* __restrict__ beta,
                                                          float* __restrict__ y, float* __restrict__ xhat,
                                                          float* __restrict__ rstd, long long rows, int cols, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const float inv_c = 1.f / (float)cols;
  for (long long r = warp0; r < rows; r += nwarps) {
    float4 v[NV];
#pragma unroll
    for (int i = 0; i < NV; i++) {
      v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if ((lane + 32 * i) * 4 < cols) v[i] = reinterpret_cast<const float4*>(x + r * cols)[lane + 32 * i];
    }
    if (RES) {
      float4 q[NV];
#pragma unroll
      for (int i = 0; i < NV; i++) {
        q[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if ((lane + 32 * i) * 4 < cols) q[i] = reinterpret_cast<const float4*>(res + r * cols)[lane + 32 * i];
      }
#pragma unroll
      for (int i = 0; i < NV; i++) { v[i].x += q[i].x; v[i].y += q[i].y; v[i].z += q[i].z; v[i].w += q[i].w; }
    }
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NV; i++) sum += v[i].x + v[i].y + v[i].z + v[i].w;
    const float mean = warp_sum(sum) * inv_c;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < NV; i++) {
      if ((lane + 32 * i) * 4 < cols) {
        v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
        sq += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
      }
    }
    const float var = warp_sum(sq) * inv_c;  // biased variance, as the reference
    const float rs = 1.f / sqrtf(var + eps);
    if (lane == 0) rstd[r] = rs;
#pragma unroll
    for (int i = 0; i < NV; i++) {
      if ((lane + 32 * i) * 4 < cols) {
        // gamma and beta stay L1-resident; reading them here keeps them out of the register file
        const float4 g = __ldg(reinterpret_cast<const float4*>(gamma) + lane + 32 * i);
        const float4 b = __ldg(reinterpret_cast<const float4*>(beta) + lane + 32 * i);
        float4 n = make_float4(v[i].x * rs, v[i].y * rs, v[i].z * rs, v[i].w * rs);
        reinterpret_cast<float4*>(xhat + r * cols)[lane + 32 * i] = n;
        reinterpret_cast<float4*>(y + r * cols)[lane + 32 * i] =
            make_float4(g.x * n.x + b.x, g.y * n.y + b.y, g.z * n.z + b.z, g.w * n.w + b.w);
      }
    }
  }
}

// The per-warp column partials of dgamma and dbeta live in dynamic shared memory (every lane owns its slots, so no
// synchronisation inside the row loop): with them in registers the kernel needed 187 registers and only one block
// fitted an SM; now two do.
template <int NV, bool ACC>
__global__ void __launch_bounds__(256, 2) layernorm_bwd_warp(const float* __restrict__ dy, const float* __restrict__ gamma,
                                                             const float* __restrict__ xhat, const float* __restrict__ rstd,
                                                             float* dx, float* dgamma, float* dbeta, long long rows, int cols) {
  extern __shared__ float4 ln_acc[];   // [2 (dgamma, dbeta)][8 warps][NV * 32] float4
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  float4* ag = ln_acc + warp * (NV * 32) + lane;
  float4* ab = ln_acc + (8 + warp) * (NV * 32) + lane;
#pragma unroll
  for (int i = 0; i < NV; i++) {
    ag[32 * i] = make_float4(0.f, 0.f, 0.f, 0.f);
    ab[32 * i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const float fc = (float)cols;
  for (long long r = warp0; r < rows; r += nwarps) {
    float4 d[NV], n[NV];
#pragma unroll
    for (int i = 0; i < NV; i++) {
      d[i] = n[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if ((lane + 32 * i) * 4 < cols) {
        d[i] = reinterpret_cast<const float4*>(dy + r * cols)[lane + 32 * i];
        n[i] = reinterpret_cast<const float4*>(xhat + r * cols)[lane + 32 * i];
      }
    }
    float sum_g = 0.f, dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; i++) {
      float4 a = ag[32 * i], bb = ab[32 * i];
      a.x += d[i].x * n[i].x; a.y += d[i].y * n[i].y; a.z += d[i].z * n[i].z; a.w += d[i].w * n[i].w;
      bb.x += d[i].x; bb.y += d[i].y; bb.z += d[i].z; bb.w += d[i].w;
      ag[32 * i] = a;
      ab[32 * i] = bb;
      float4 g = make_float4(0.f, 0.f, 0.f, 0.f);   // gamma stays in L1: re-read per row instead of held in registers
      if ((lane + 32 * i) * 4 < cols) g = __ldg(reinterpret_cast<const float4*>(gamma) + lane + 32 * i);
      d[i].x *= g.x; d[i].y *= g.y; d[i].z *= g.z; d[i].w *= g.w;  // grad wrt xhat
      sum_g += d[i].x + d[i].y + d[i].z + d[i].w;
      dot += d[i].x * n[i].x + d[i].y * n[i].y + d[i].z * n[i].z + d[i].w * n[i].w;
    }
    sum_g = warp_sum(sum_g);
    dot = warp_sum(dot);
    if (dx) {
      const float k = rstd[r] / fc;
      float4 old[ACC ? NV : 1];
      if (ACC) {  // all old values requested before the first store of the row
#pragma unroll
        for (int i = 0; i < NV; i++) {
          old[ACC ? i : 0] = make_float4(0.f, 0.f, 0.f, 0.f);
          if ((lane + 32 * i) * 4 < cols) old[ACC ? i : 0] = (reinterpret_cast<const float4*>(dx + r * cols))[lane + 32 * i];
        }
      }
#pragma unroll
      for (int i = 0; i < NV; i++) {
        if ((lane + 32 * i) * 4 < cols) {
          float4 o = make_float4(k * (fc * d[i].x - sum_g - n[i].x * dot), k * (fc * d[i].y - sum_g - n[i].y * dot),
                                 k * (fc * d[i].z - sum_g - n[i].z * dot), k * (fc * d[i].w - sum_g - n[i].w * dot));
          if (ACC) { o.x += old[ACC ? i : 0].x; o.y += old[ACC ? i : 0].y; o.z += old[ACC ? i : 0].z; o.w += old[ACC ? i : 0].w; }
          reinterpret_cast<float4*>(dx + r * cols)[lane + 32 * i] = o;
        }
      }
    }
  }
  // column partials of the 8 warps -> one atomic per column per block
  __syncthreads();
  const float* accf = reinterpret_cast<const float*>(ln_acc);
  for (int pass = 0; pass < 2; pass++) {
    float* dst = pass == 0 ? dgamma : dbeta;
    if (!dst) continue;
    for (int c = threadIdx.x; c < NV * 128; c += 256) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 8; w++) t += accf[(size_t)(pass * 8 + w) * (NV * 128) + c];
      if (c < cols) atomicAdd(dst + c, t);
    }
  }
}

__global__ void __launch_bounds__(256) layernorm_fwd_block(const float* __restrict__ x, const float* __restrict__ res,
                                                           const float* __restrict__ gamma, const float* __restrict__ beta,
                                                           float* __restrict__ y, float* __restrict__ xhat,
                                                           float* __restrict__ rstd, long long rows, int cols, float eps) {
  __shared__ float red[8];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    float s = 0.f;
    for (int c = threadIdx.x; c < cols; c += 256) s += x[r * cols + c] + (res ? res[r * cols + c] : 0.f);
    const float mean = block_sum(s, red) / cols;
    float sq = 0.f;
    for (int c = threadIdx.x; c < cols; c += 256) {
      float d = x[r * cols + c] + (res ? res[r * cols + c] : 0.f) - mean;
      sq += d * d;
    }
    const float rs = 1.f / sqrtf(block_sum(sq, red) / cols + eps);
    if (threadIdx.x == 0) rstd[r] = rs;
    for (int c = threadIdx.x; c < cols; c += 256) {
      float n = (x[r * cols + c] + (res ? res[r * cols + c] : 0.f) - mean) * rs;
      xhat[r * cols + c] = n;
      y[r * cols + c] = gamma[c] * n + beta[c];
    }
  }
}
__global__ void __launch_bounds__(256) layernorm_bwd_block(const float* __restrict__ dy, const float* __restrict__ gamma,
                                                           const float* __restrict__ xhat, const float* __restrict__ rstd,
                                                           float* dx, float* dgamma, float* dbeta, long long rows, int cols,
                                                           int accumulate_dx) {
  __shared__ float red[8];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    float sum_g = 0.f, dot = 0.f;
    for (int c = threadIdx.x; c < cols; c += 256) {
      const float d = dy[r * cols + c], n = xhat[r * cols + c];
      if (dgamma) atomicAdd(dgamma + c, d * n);
      if (dbeta) atomicAdd(dbeta + c, d);
      sum_g += d * gamma[c];
      dot += d * gamma[c] * n;
    }
    sum_g = block_sum(sum_g, red);
    dot = block_sum(dot, red);
    if (dx) {
      const float k = rstd[r] / cols;
      for (int c = threadIdx.x; c < cols; c += 256) {
        float o = k * (cols * dy[r * cols + c] * gamma[c] - sum_g - xhat[r * cols + c] * dot);
        dx[r * cols + c] = accumulate_dx ? dx[r * cols + c] + o : o;
      }
    }
  }
}

// --------------------------------------------------------------- softmax cross-entropy
// One block per row, online (max, sum) in a single read, then a second read (L2-resident for
// rows of this size) that writes the gradient.  Per-row losses go to scratch and are summed in
// double by a single block, so the result does not depend on the launch geometry.
// A label outside [0, cols) is never used as an index: the row then contributes no loss and no one-hot term (its
// gradient is the plain softmax) and the status block records FML_BAD_INDEX_LABEL.
__global__ void __launch_bounds__(256) xent_kernel(const float* z, const int* __restrict__ labels, float* dz,
                                                   float* __restrict__ row_loss, long long rows, int cols, float inv_count,
                                                   int* status) {
  __shared__ float red[8];
  __shared__ float zl_s;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* zr = z + r * cols;
    float mx = NEG_INF, s = 0.f;
    for (int c = threadIdx.x; c < cols; c += 256) {
      const float v = zr[c];
      if (v > mx) { s = s * expf(mx - v); mx = v; }
      s += expf(v - mx);
    }
    const float bm = block_max(mx, red);
    s = (mx == NEG_INF) ? 0.f : s * expf(mx - bm);
    s = block_sum(s, red);
    const int lab = labels[r];
    const bool lab_ok = (unsigned)lab < (unsigned)cols;
    if (threadIdx.x == 0) {
      zl_s = lab_ok ? zr[lab] : 0.f;
      if (!lab_ok) fml_flag_bad_index(status, FML_BAD_INDEX_LABEL);
    }
    __syncthreads();
    const float zl = zl_s;
    if (threadIdx.x == 0) row_loss[r] = lab_ok ? -(zl - bm - logf(s)) * inv_count : 0.f;
    if (dz) {
      float* dr = dz + r * cols;
      for (int c = threadIdx.x; c < cols; c += 256) dr[c] = (expf(zr[c] - bm) / s - (c == lab ? 1.f : 0.f)) * inv_count;
    }
    __syncthreads();
  }
}

// Wide rows (vocabulary-sized logits): one 1024-thread block per row keeps the whole row in registers
// (NV float4 per thread, all loads issued before the first use), so the logits are read from HBM exactly once
// and the gradient written once: 8 bytes per element.  Two block reductions (max, sum of 2^(k(v - max))).
// COLSUM: the block also sums the gradient rows it produces, column by column, in dynamic shared memory (every
// thread owns its columns, so no synchronisation) and leaves one partial row per block in `colpart`: the bias
// gradient of the layer that produced the logits, without a second pass over the gradient.
template <int NV, bool COLSUM>
__global__ void __launch_bounds__(1024) xent_rowreg_kernel(const float* z, const int* __restrict__ labels,
                                                           float* dz /* may alias z */, float* __restrict__ row_loss,
                                                           long long rows, int cols, float inv_count, float* __restrict__ colpart,
                                                           int* status) {
  extern __shared__ float4 colacc[];   // [cols / 4], COLSUM only
  __shared__ float red[32];
  __shared__ float bcast[3];
  if (COLSUM) {
#pragma unroll
    for (int i = 0; i < NV; i++) {
      const int c4 = threadIdx.x + 1024 * i;
      if (c4 * 4 < cols) colacc[c4] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr float LOG2E = 1.4426950408889634f;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const float4* zr = reinterpret_cast<const float4*>(z + r * cols);
    float4 v[NV];
#pragma unroll
    for (int i = 0; i < NV; i++) {
      const int c4 = threadIdx.x + 1024 * i;
      v[i] = make_float4(NEG_INF, NEG_INF, NEG_INF, NEG_INF);
      if (c4 * 4 < cols) v[i] = zr[c4];
    }
    const int lab = labels[r];
    const bool lab_ok = (unsigned)lab < (unsigned)cols;   // otherwise no thread owns the label's column below
    if (!lab_ok && threadIdx.x == 0) fml_flag_bad_index(status, FML_BAD_INDEX_LABEL);
    float mx = NEG_INF;
#pragma unroll
    for (int i = 0; i < NV; i++) {
      mx = fmaxf(mx, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
      const int d = lab - (threadIdx.x + 1024 * i) * 4;  // the owner of the label's column publishes its logit
      if (d >= 0 && d < 4) bcast[2] = d == 0 ? v[i].x : d == 1 ? v[i].y : d == 2 ? v[i].z : v[i].w;
    }
    mx = warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    if (warp == 0) {
      const float t = warp_max(red[lane]);
      if (lane == 0) bcast[0] = t;
    }
    __syncthreads();
    const float bm = bcast[0];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; i++) {  // 2^(-inf) = 0 for the padding beyond cols
      v[i].x = fml_exp2_ftz((v[i].x - bm) * LOG2E); v[i].y = fml_exp2_ftz((v[i].y - bm) * LOG2E);
      v[i].z = fml_exp2_ftz((v[i].z - bm) * LOG2E); v[i].w = fml_exp2_ftz((v[i].w - bm) * LOG2E);
      s += v[i].x + v[i].y + v[i].z + v[i].w;
    }
    s = warp_sum(s);
    if (lane == 0) red[warp] = s;   // all reads of red[] for the max finished before the barrier above
    __syncthreads();
    if (warp == 0) {
      const float t = warp_sum(red[lane]);
      if (lane == 0) bcast[1] = t;
    }
    __syncthreads();
    const float tot = bcast[1];
    if (threadIdx.x == 0) row_loss[r] = lab_ok ? -(bcast[2] - bm - logf(tot)) * inv_count : 0.f;
    if (dz) {
      const float k = inv_count / tot;
      float4* dr = reinterpret_cast<float4*>(dz + r * cols);
#pragma unroll
      for (int i = 0; i < NV; i++) {
        const int c4 = threadIdx.x + 1024 * i;
        if (c4 * 4 < cols) {
          float4 o = make_float4(v[i].x * k, v[i].y * k, v[i].z * k, v[i].w * k);
          const int d = lab - c4 * 4;
          if (d == 0) o.x -= inv_count; else if (d == 1) o.y -= inv_count; else if (d == 2) o.z -= inv_count; else if (d == 3) o.w -= inv_count;
          dr[c4] = o;
          if (COLSUM) {
            float4 a = colacc[c4];
            a.x += o.x; a.y += o.y; a.z += o.z; a.w += o.w;
            colacc[c4] = a;
          }
        }
      }
    }
    __syncthreads();  // bcast / red are rewritten by the next row
  }
  if (COLSUM) {
#pragma unroll
    for (int i = 0; i < NV; i++) {
      const int c4 = threadIdx.x + 1024 * i;
      if (c4 * 4 < cols) reinterpret_cast<float4*>(colpart + (size_t)blockIdx.x * cols)[c4] = colacc[c4];
    }
  }
}

__global__ void __launch_bounds__(256) mse_kernel(const float* __restrict__ p, const float* __restrict__ t, float* dp,
                                                  double* __restrict__ partial, long long n, float k) {
  __shared__ double red[8];
  double acc = 0.0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float e = p[i] - t[i];
    acc += (double)e * e;
    if (dp) dp[i] = k * e;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double tsum = 0.0;
    for (int w = 0; w < 8; w++) tsum += red[w];
    partial[blockIdx.x] = tsum;
  }
}

template <class T>
__global__ void __launch_bounds__(256) final_sum_kernel(const T* __restrict__ part, long long n, double mul, float* out) {
  __shared__ double red[8];
  double acc = 0.0;
  for (long long i = threadIdx.x; i < n; i += 256) acc += (double)part[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double tsum = 0.0;
    for (int w = 0; w < 8; w++) tsum += red[w];
    *out += (float)(tsum * mul);
  }
}

inline int warp_row_blocks(fml_ctx* ctx, long long rows) {
  long long b = (rows + 7) / 8;  // 8 warps per block, one row per warp per trip
  return (int)std::max<long long>(1, std::min<long long>(b, (long long)ctx->sm_count * 8));
}
inline int block_row_blocks(fml_ctx* ctx, long long rows) {
  return (int)std::max<long long>(1, std::min<long long>(rows, (long long)ctx->sm_count * 8));
}

#define DISPATCH_NV(cols, CALL)            \
  do {                                     \
    if ((cols) <= 128) { CALL(1); }        \
    else if ((cols) <= 256) { CALL(2); }   \
    else if ((cols) <= 512) { CALL(4); }   \
    else if ((cols) <= 1024) { CALL(8); }  \
    else { CALL(16); }                     \
  } while (0)

}  // namespace

extern "C" {

int32_t fml_softmax_rows_fwd(fml_ctx* ctx, const float* x, float* y, int64_t rows, int32_t cols, float scale,
                             int32_t causal_period) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, x && y && rows > 0 && cols > 0, "fml_softmax_rows_fwd: bad arguments");
  if (cols % 4 == 0 && cols <= 2048 && al16(x) && al16(y)) {
#define CALL(NV) softmax_fwd_warp<NV><<<warp_row_blocks(ctx, rows), 256, 0, ctx->stream>>>(x, y, rows, cols, scale, causal_period)
    DISPATCH_NV(cols, CALL);
#undef CALL
  } else {
    softmax_fwd_block<<<block_row_blocks(ctx, rows), 256, 0, ctx->stream>>>(x, y, rows, cols, scale, causal_period);
  }
  FML_LAUNCH_CHECK(ctx, "softmax_fwd");
  return FML_OK;
}

int32_t fml_softmax_rows_bwd(fml_ctx* ctx, const float* y, const float* dy, float* dx, int64_t rows, int32_t cols,
                             float scale, int32_t accumulate) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, y && dy && dx && rows > 0 && cols > 0, "fml_softmax_rows_bwd: bad arguments");
  if (cols % 4 == 0 && cols <= 2048 && al16(y) && al16(dy) && al16(dx)) {
#define CALL(NV)                                                                                             \
  do {                                                                                                       \
    if (accumulate)                                                                                          \
      softmax_bwd_warp<NV, true><<<warp_row_blocks(ctx, rows), 256, 0, ctx->stream>>>(y, dy, dx, rows, cols, scale);  \
    else                                                                                                     \
      softmax_bwd_warp<NV, false><<<warp_row_blocks(ctx, rows), 256, 0, ctx->stream>>>(y, dy, dx, rows, cols, scale); \
  } while (0)
    DISPATCH_NV(cols, CALL);
#undef CALL
  } else {
    softmax_bwd_block<<<block_row_blocks(ctx, rows), 256, 0, ctx->stream>>>(y, dy, dx, rows, cols, scale, accumulate);
  }
  FML_LAUNCH_CHECK(ctx, "softmax_bwd");
  return FML_OK;
}

int32_t fml_layernorm_fwd(fml_ctx* ctx, const float* x, const float* residual, const float* gamma, const float* beta,
                          float* y, float* xhat, float* rstd, int64_t rows, int32_t cols, float eps) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, x && gamma && beta && y && xhat && rstd && rows > 0 && cols > 0, "fml_layernorm_fwd: bad arguments");
  if (cols % 4 == 0 && cols <= 2048 && al16(x) && al16(y) && al16(xhat) && al16(gamma) && al16(beta) &&
      (!residual || al16(residual))) {
#define CALL(NV)                                                                                                              \
  do {                                                                                                                        \
    if (residual)                                                                                                             \
      layernorm_fwd_warp<NV, true><<<warp_row_blocks(ctx, rows), 256, 0, ctx->stream>>>(x, residual, gamma, beta, y, xhat, rstd, rows, cols, eps); \
    else                                                                                                                      \
      layernorm_fwd_warp<NV, false><<<warp_row_blocks(ctx, rows), 256, 0, ctx->stream>>>(x, residual, gamma, beta, y, xhat, rstd, rows, cols, eps); \
  } while (0)
    DISPATCH_NV(cols, CALL);
#undef CALL
  } else {
    layernorm_fwd_block<<<block_row_blocks(ctx, rows), 256, 0, ctx->stream>>>(x, residual, gamma, beta, y, xhat, rstd, rows, cols, eps);
  }
  FML_LAUNCH_CHECK(ctx, "layernorm_fwd");
  return FML_OK;
}

int32_t fml_layernorm_bwd(fml_ctx* ctx, const float* dy, const float* gamma, const float* xhat, const float* rstd,
                          float* dx, float* dgamma, float* dbeta, int64_t rows, int32_t cols, int32_t accumulate_dx) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, dy && gamma && xhat && rstd && rows > 0 && cols > 0, "fml_layernorm_bwd: bad arguments");
  if (cols % 4 == 0 && cols <= 1024 && al16(dy) && al16(xhat) && al16(gamma) && (!dx || al16(dx))) {
    // fewer, fatter blocks: every block ends with one atomic per column
    const int blocks = (int)std::max<long long>(1, std::min<long long>((rows + 7) / 8, (long long)ctx->sm_count * 2));
#define CALL(NV)                                                                                                     \
  do {                                                                                                               \
    const size_t sm = (size_t)2 * 8 * NV * 128 * sizeof(float);                                                      \
    FML_ONCE_PER_DEVICE(ctx, {                                                                                       \
      FML_CUDA(ctx, cudaFuncSetAttribute(layernorm_bwd_warp<NV, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));  \
      FML_CUDA(ctx, cudaFuncSetAttribute(layernorm_bwd_warp<NV, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm)); \
    });                                                                                                              \
    if (accumulate_dx && dx)                                                                                         \
      layernorm_bwd_warp<NV, true><<<blocks, 256, sm, ctx->stream>>>(dy, gamma, xhat, rstd, dx, dgamma, dbeta, rows, cols);  \
    else                                                                                                             \
      layernorm_bwd_warp<NV, false><<<blocks, 256, sm, ctx->stream>>>(dy, gamma, xhat, rstd, dx, dgamma, dbeta, rows, cols); \
  } while (0)
    if (cols <= 128) { CALL(1); } else if (cols <= 256) { CALL(2); } else if (cols <= 512) { CALL(4); } else { CALL(8); }
#undef CALL
  } else {
    layernorm_bwd_block<<<block_row_blocks(ctx, rows), 256, 0, ctx->stream>>>(dy, gamma, xhat, rstd, dx, dgamma, dbeta, rows, cols, accumulate_dx);
  }
  FML_LAUNCH_CHECK(ctx, "layernorm_bwd");
  return FML_OK;
}

static int32_t softmax_xent_impl(fml_ctx* ctx, const float* z, const int32_t* labels, float* dz, float* loss_sum, int64_t rows,
                                 int32_t cols, float inv_count, float* dbias) {
  const bool wide = cols >= 4096 && cols <= 32768 && cols % 4 == 0 && al16(z) && (!dz || al16(dz));
  const int blocks = (int)std::max<long long>(1, std::min<long long>(rows, (long long)ctx->sm_count * 2));
  const bool fuse = dbias && dz && wide;
  const size_t loss_bytes = ((size_t)rows * sizeof(float) + 255) & ~(size_t)255;
  int32_t rc = fml_ensure_workspace(ctx, loss_bytes + (fuse ? (size_t)blocks * cols * sizeof(float) : 0));
  if (rc) return rc;
  float* row_loss = reinterpret_cast<float*>(ctx->ws);
  float* colpart = reinterpret_cast<float*>(ctx->ws + loss_bytes);
  if (wide) {
#define XENT(NV)                                                                                                              \
  do {                                                                                                                        \
    if (fuse) {                                                                                                               \
      FML_ONCE_PER_DEVICE(ctx, {                                                                                              \
        FML_CUDA(ctx, cudaFuncSetAttribute(xent_rowreg_kernel<NV, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768 * 4)); \
      });                                                                                                                     \
      xent_rowreg_kernel<NV, true><<<blocks, 1024, (size_t)cols * 4, ctx->stream>>>(z, labels, dz, row_loss, rows, cols, inv_count, colpart, ctx->d_status); \
    } else {                                                                                                                  \
      xent_rowreg_kernel<NV, false><<<blocks, 1024, 0, ctx->stream>>>(z, labels, dz, row_loss, rows, cols, inv_count, nullptr, ctx->d_status); \
    }                                                                                                                         \
  } while (0)
    if (cols <= 8192) XENT(2);
    else if (cols <= 16384) XENT(4);
    else XENT(8);
#undef XENT
  } else {
    xent_kernel<<<block_row_blocks(ctx, rows), 256, 0, ctx->stream>>>(z, labels, dz, row_loss, rows, cols, inv_count, ctx->d_status);
  }
  final_sum_kernel<float><<<1, 256, 0, ctx->stream>>>(row_loss, rows, 1.0, loss_sum);
  FML_LAUNCH_CHECK(ctx, "xent_kernel");
  if (dbias) {
    FML_REQUIRE(ctx, dz, "fml_softmax_xent_dbias: the bias gradient needs dz");
    // one partial row per block (fused) or the gradient itself (other shapes), summed into dbias
    return fuse ? fml_col_sum(ctx, colpart, dbias, blocks, cols, 1) : fml_col_sum(ctx, dz, dbias, rows, cols, 1);
  }
  return FML_OK;
}

int32_t fml_softmax_xent(fml_ctx* ctx, const float* z, const int32_t* labels, float* dz, float* loss_sum, int64_t rows,
                         int32_t cols, float inv_count) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, z && labels && loss_sum && rows > 0 && cols > 0, "fml_softmax_xent: bad arguments");
  return softmax_xent_impl(ctx, z, labels, dz, loss_sum, rows, cols, inv_count, nullptr);
}

int32_t fml_softmax_xent_dbias(fml_ctx* ctx, const float* z, const int32_t* labels, float* dz, float* loss_sum, int64_t rows,
                               int32_t cols, float inv_count, float* dbias) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, z && labels && dz && loss_sum && dbias && rows > 0 && cols > 0, "fml_softmax_xent_dbias: bad arguments");
  return softmax_xent_impl(ctx, z, labels, dz, loss_sum, rows, cols, inv_count, dbias);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free softmax cross-entropy.
//
// fml_softmax_xent keeps its per-row losses in the context's scratch arena, which it grows with
// cudaMalloc when a larger batch arrives.  Some callers must never reach an allocator: a host
// framework whose own caching allocator already owns all of HBM (a cudaMalloc there fails or
// fragments its pool), a serving loop that cannot afford the device-wide synchronisation cudaMalloc
// and cudaFree imply, or code that runs while the allocator is locked.  For them the per-row
// losses live in the fixed array below, which every GPU that loads this library holds until the
// process exits (FML_XENT_STATIC_MAX_ROWS floats = 256 KiB).
//
// In host code the name `g_xent_static_rows` is only a stand-in for the symbol, not a device
// address, so the set-up asks the runtime for the address once per device (with that device
// current) and the launches pass the pointer it returned.
__device__ __align__(256) float g_xent_static_rows[FML_XENT_STATIC_MAX_ROWS];

namespace {
constexpr int kMaxDevices = 64;
float* g_xent_static_ptr[kMaxDevices] = {};
int g_xent_static_sms[kMaxDevices] = {};
}  // namespace

int32_t fml_softmax_xent_static(fml_ctx* ctx, const float* z, const int32_t* labels, float* dz, float* loss_sum,
                                int64_t rows, int32_t cols, float inv_count) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, z && labels && loss_sum && rows > 0 && cols > 0, "fml_softmax_xent_static: bad arguments");
  if (rows > FML_XENT_STATIC_MAX_ROWS)
    return fml_fail(ctx, FML_ERR_OOM,
                    "fml_softmax_xent_static: " + std::to_string((long long)rows) + " rows exceed the fixed scratch of " +
                        std::to_string(FML_XENT_STATIC_MAX_ROWS) + " rows; split the batch or use fml_softmax_xent");
  const int dev = ctx->device;
  FML_REQUIRE(ctx, dev >= 0 && dev < kMaxDevices, "fml_softmax_xent_static: device ordinal out of range");
  if (!g_xent_static_ptr[dev]) {
    // first call on this device: resolve the symbol (no allocation; do this before any stream capture)
    FML_CUDA(ctx, cudaSetDevice(dev));
    float* ptr = nullptr;
    FML_CUDA(ctx, cudaGetSymbolAddress((void**)&ptr, g_xent_static_rows));
    FML_REQUIRE(ctx, ptr != nullptr, "fml_softmax_xent_static: the scratch symbol has no device address");
    g_xent_static_sms[dev] = ctx->sm_count;
    g_xent_static_ptr[dev] = ptr;
  }
  float* row_loss = g_xent_static_ptr[dev];
  // every row slot read by the final sum is written by this launch first, so nothing needs clearing
  const int blocks = (int)std::max<long long>(1, std::min<long long>(rows, (long long)g_xent_static_sms[dev] * 8));
  xent_kernel<<<blocks, 256, 0, ctx->stream>>>(z, labels, dz, row_loss, rows, cols, inv_count, ctx->d_status);
  final_sum_kernel<float><<<1, 256, 0, ctx->stream>>>(row_loss, rows, 1.0, loss_sum);
  FML_LAUNCH_CHECK(ctx, "xent_kernel (static scratch)");
  return FML_OK;
}

int32_t fml_mse(fml_ctx* ctx, const float* p, const float* t, float* dp, float* loss_sum, int64_t n, float upstream) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, p && t && loss_sum && n > 0, "fml_mse: bad arguments");
  const int blocks = (int)std::max<long long>(1, std::min<long long>((n + 255) / 256, (long long)ctx->sm_count * 4));
  int32_t rc = fml_ensure_workspace(ctx, (size_t)blocks * sizeof(double));
  if (rc) return rc;
  double* partial = reinterpret_cast<double*>(ctx->ws);
  mse_kernel<<<blocks, 256, 0, ctx->stream>>>(p, t, dp, partial, n, upstream * 2.f / (float)n);
  final_sum_kernel<double><<<1, 256, 0, ctx->stream>>>(partial, blocks, 1.0 / (double)n, loss_sum);
  FML_LAUNCH_CHECK(ctx, "mse_kernel");
  return FML_OK;
}

}  // extern "C"
