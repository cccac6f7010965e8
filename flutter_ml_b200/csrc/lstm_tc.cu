// LSTM forward recurrence as ONE cooperative kernel for all time steps.
//
// Launched once per sequence batch instead of once per step: the per-step launch, TMEM allocation, barrier set-up
// and tear-down of a tensor-core kernel cost about 5 us, more than the step's arithmetic.  Here every CTA owns NC = 32
// consecutive gate columns (8 hidden units x f, i, c~, o of the gate-interleaved weight) for the whole sequence:
//   - its slice of the recurrent weight Wh' [NC x H] is loaded into shared memory once and stays there;
//   - per step the producer streams h_{t-1} [128 x H] through a TMA ring, the issuer accumulates
//     Z[128 x NC] = h_{t-1} . Wh'^T in TMEM, and the four gate warps (thread = batch row) add the input projection
//     (prefetched before the product finishes), apply the gate functions and the cell update, keep c in REGISTERS
//     across steps, and write gates, c_t and their 8 columns of h_t;
//   - a grid-wide barrier (one atomic counter, bounded spin) separates the steps: h_t is complete before any CTA
//     loads it.  The launch is cooperative, so all CTAs are resident together or the launch fails.
// Generic-proxy stores of h_t by other CTAs are read through TMA (async proxy): writers fence with __threadfence and
// fence.proxy.async before they signal, the loader fences again after it has observed the counter.
// Requirements: batch <= 128, H % 32 == 0, 4H / 32 <= number of SMs, the weight slice (128 H bytes) plus the ring fits
// in shared memory; other shapes use the per-step kernels.  Reference: LSTMLayer.forward lib/layertypes/lstmLayer.dart:112-150.
#include <algorithm>
#include <cstdio>
#include <cstdlib>

#include "common.cuh"
#include "tc_ptx.cuh"

int32_t fml_tc_make_tmap(fml_ctx* ctx, const float* base, int64_t cols, int64_t rows, int64_t ld, int64_t nb1, int64_t nb2,
                         int64_t s1, int64_t s2, int box_c, int box_r, bool mn_major, int blocks, CUtensorMap* out);

using namespace fml_tc;

namespace {

constexpr int NC = 32;            // gate columns per CTA
constexpr int LT_THREADS = 192;   // producer warp, issuer warp, 4 gate warps
constexpr int A_STAGE = 128 * 32 * 4;   // one k-block of h: 128 rows x 32 floats
constexpr int MAX_RING = 8;

struct LstmPParams {
  int T, B, H, kblocks, ring;
  uint32_t w_bytes;          // NC * H * 4
  const float* xproj;        // [T*B][4H] input projection + bias, gate-interleaved
  float* gates;              // [T][B][4H]
  float* cells;              // [T+1][B][H]
  float* hs;                 // [T+1][B][H]
  unsigned int* gbar;        // grid barrier counter (zeroed before the launch)
  int fast_math;
  int* status;
  long long* prof;           // -DFML_LSTM_PROFILE builds: clock64 stamps of one step of CTA 0, else NULL
};

#ifdef FML_LSTM_PROFILE
#define LT_STAMP(k) do { if (p.prof && blockIdx.x == 0 && t == 64) p.prof[k] = clock64(); } while (0)
#else
#define LT_STAMP(k) do { } while (0)
#endif

enum { L_WFULL = 0, L_ACCFULL = 1, L_ACCEMPTY = 2, L_STEPDONE = 3, L_FULL = 4, L_EMPTY = 4 + MAX_RING, L_COUNT = 4 + 2 * MAX_RING };

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(LT_THREADS, 1)
lstm_fwd_persistent_kernel(const __grid_constant__ CUtensorMap tmH, const __grid_constant__ CUtensorMap tmW, const LstmPParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t off_ring = (p.w_bytes + 1023u) & ~1023u;
  const uint32_t off_bar = off_ring + (uint32_t)p.ring * A_STAGE;
  auto bar = [&](int i) { return smem_base + off_bar + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + off_bar + 8 * L_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * NC;   // first gate column of this CTA

  if (threadIdx.x == 0) {
    for (int i = 0; i < L_COUNT; i++) mbar_init(bar(i), (i == L_ACCEMPTY || i == L_STEPDONE) ? 128u : 1u);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(32u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer + grid barrier
    if (lane == 0) {
      // the weight slice, once: k-block kb = NC rows x 128 B
      mbar_expect_tx(bar(L_WFULL), p.w_bytes);
      for (int kb = 0; kb < p.kblocks; kb++) tma_load_4d(smem_base + kb * (NC * 128), &tmW, bar(L_WFULL), kb * 32, n0, 0, 0);
      bool ok = true;
      uint32_t g = 0;   // k-blocks streamed so far
      for (int t = 0; t < p.T && ok; t++) {
        if (t > 0) {
          // every CTA has written its columns of h_t (= hs[t]) before anyone loads them
          ok = mbar_wait(bar(L_STEPDONE), (uint32_t)(t - 1) & 1u, abort_flag, p.status, 51);
          if (!ok) break;
          LT_STAMP(0);
          // one release-add without a return value: the gate warps' stores of h_t (each behind its own fence, observed by this
          // thread through the mbarrier) are ordered before it, and nothing waits for the counter's old value
          asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.gbar) : "memory");
          const unsigned int target = (unsigned int)t * gridDim.x;
          const unsigned long long t0 = globaltimer_ns();
          while (ld_acquire_gpu(p.gbar) < target) {
            if (*abort_flag || globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
              *abort_flag = 1;
              atomicCAS(p.status, 0, 52);
              ok = false;
              break;
            }
          }
          if (!ok) break;
          asm volatile("fence.proxy.async.global;" ::: "memory");
          LT_STAMP(1);
        }
        for (int kb = 0; kb < p.kblocks && ok; kb++, g++) {
          const int s = (int)(g % (uint32_t)p.ring);
          const uint32_t ph = (g / (uint32_t)p.ring) & 1u;
          ok = mbar_wait(bar(L_EMPTY + s), ph ^ 1u, abort_flag, p.status, 53);
          if (!ok) break;
          mbar_expect_tx(bar(L_FULL + s), A_STAGE);
          // (Every CTA walks the k-blocks of h_{t-1} in the same order.  Starting each CTA at its own block was measured:
          // slower, 1.64 against 1.45 ms for 128 steps; CTAs asking for the same lines at the same time help each other.)
          tma_load_4d(smem_base + off_ring + s * A_STAGE, &tmH, bar(L_FULL + s), kb * 32, t * p.B, 0, 0);
        }
        LT_STAMP(2);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(NC >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      bool ok = mbar_wait(bar(L_WFULL), 0, abort_flag, p.status, 54);
      uint32_t g = 0;
      for (int t = 0; t < p.T && ok; t++) {
        ok = mbar_wait(bar(L_ACCEMPTY), ((uint32_t)t & 1u) ^ 1u, abort_flag, p.status, 55);   // gate warps have read step t-1
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < p.kblocks && ok; kb++, g++) {
          const int s = (int)(g % (uint32_t)p.ring);
          const uint32_t ph = (g / (uint32_t)p.ring) & 1u;
          ok = mbar_wait(bar(L_FULL + s), ph, abort_flag, p.status, 56);
          if (!ok) break;
          if (kb == 0) LT_STAMP(3);
          tc_fence_after();
          const uint64_t ad = make_smem_desc(smem_base + off_ring + s * A_STAGE, 16u, 1024u, 2u);
          const uint64_t bd = make_smem_desc(smem_base + kb * (NC * 128), 16u, 1024u, 2u);
#pragma unroll
          for (int k = 0; k < 4; k++) umma_tf32(tmem_base, ad + 2u * k, bd + 2u * k, idesc, (kb | k) ? 1u : 0u);
          umma_commit(bar(L_EMPTY + s));
        }
        if (ok) umma_commit(bar(L_ACCFULL));
        LT_STAMP(4);
      }
    }
  } else {
    // ------------------------------------------------------------------ gate warps: thread = batch row
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    const bool active = row < p.B;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q4 * 32) << 16);
    const int N = 4 * p.H, u0 = n0 >> 2;   // first hidden unit of this CTA
    float c[NC / 4];
#pragma unroll
    for (int i = 0; i < NC / 4; i++) c[i] = 0.f;   // c_0 = 0 (lstmLayer.dart:115)
    bool ok = true;
    uint32_t v[32];
    for (int t = 0; t < p.T && ok; t++) {
      // the input projection of this step does not depend on the recurrence: request it before waiting
      float4 xa[NC / 4];
      const long long po = ((long long)t * p.B + row) * N + n0;
#pragma unroll
      for (int i = 0; i < NC / 4; i++) xa[i] = active ? __ldg(reinterpret_cast<const float4*>(p.xproj + po) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      ok = mbar_wait(bar(L_ACCFULL), (uint32_t)t & 1u, abort_flag, p.status, 57);
      if (!ok) break;
      if (threadIdx.x == 64) LT_STAMP(5);
      tc_fence_after();
      tmem_ld32(lane_addr, v);
      tmem_ld_wait();
      if (threadIdx.x == 64) LT_STAMP(6);
      tc_fence_before();
      mbar_arrive(bar(L_ACCEMPTY));
      float hn[NC / 4];
      float4 gt[NC / 4];
#pragma unroll
      for (int i = 0; i < NC / 4; i++) {
        const float zf = __uint_as_float(v[4 * i]) + xa[i].x, zi = __uint_as_float(v[4 * i + 1]) + xa[i].y;
        const float zg = __uint_as_float(v[4 * i + 2]) + xa[i].z, zo = __uint_as_float(v[4 * i + 3]) + xa[i].w;
        float f, ig, g, o;
        if (p.fast_math) {
          f = fml_sigmoid_fast(zf); ig = fml_sigmoid_fast(zi); g = fml_tanh_fast(zg); o = fml_sigmoid_fast(zo);
        } else {
          f = fml_sigmoid(zf); ig = fml_sigmoid(zi); g = fml_tanh_ref(zg); o = fml_sigmoid(zo);
        }
        c[i] = f * c[i] + ig * g;
        hn[i] = o * (p.fast_math ? fml_tanh_fast(c[i]) : fml_tanh_ref(c[i]));
        gt[i] = make_float4(f, ig, g, o);
      }
      if (threadIdx.x == 64) LT_STAMP(7);
      const long long ho = ((long long)(t + 1) * p.B + row) * p.H + u0;
      // h_t first: it is the only output the next step waits for.  Make it visible to the other CTAs' TMA loads and
      // report the step; the saved gates and cells (read by the backward pass only) are stored off the critical path.
      if (active) {
#pragma unroll
        for (int i = 0; i < NC / 4; i += 4) *reinterpret_cast<float4*>(p.hs + ho + i) = make_float4(hn[i], hn[i + 1], hn[i + 2], hn[i + 3]);
      }
      __threadfence();
      asm volatile("fence.proxy.async.global;" ::: "memory");
      mbar_arrive(bar(L_STEPDONE));
      if (threadIdx.x == 64) LT_STAMP(8);
      if (active) {
#pragma unroll
        for (int i = 0; i < NC / 4; i++) reinterpret_cast<float4*>(p.gates + po)[i] = gt[i];
#pragma unroll
        for (int i = 0; i < NC / 4; i += 4) *reinterpret_cast<float4*>(p.cells + ho + i) = make_float4(c[i], c[i + 1], c[i + 2], c[i + 3]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32u) : "memory");
  }
}


// ------------------------------------------------------------------------------------------------------------
// The same recurrence with the contraction over H split between the two CTAs of a cluster.  Measured on the kernel above
// (H 512, batch 128; clock64 stamps of one step, -DFML_LSTM_PROFILE): of the 19 800 cycles of a step, 10 000 pass between
// the first block of h_{t-1} arriving and the last product being issued, because every CTA pulls all 256 KiB of h_{t-1}
// through its one L2 port (26 bytes per clock) for 64 instructions of N = 32; the grid barrier takes 4000, the gate
// arithmetic 2350, storing h and reporting 1400.  Here a pair of CTAs owns the 32 gate columns: each loads HALF of the
// k-blocks of h_{t-1} (and keeps half of the weight slice), issues 32 instructions, and finalises 16 of the 32 columns
// (4 hidden units): it keeps those 16 columns of its partial sums in registers, parks the other 16 in its shared memory
// for the partner, and adds the partner's 16 through distributed shared memory.  Twice the CTAs (8H / 32, 128 of 148 SMs
// at H = 512), half the bytes, instructions and gate arithmetic per CTA.
constexpr int PART_LD = 20;   // floats per row of the parked half (16 + padding: rows 80 bytes apart spread over the banks)
constexpr int LP_THREADS = 320;   // paired kernel: producer warp, issuer warp, 8 gate warps
enum { P_WFULL = 0, P_ACCFULL = 1, P_ACCEMPTY = 2, P_STEPDONE = 3, P_PARTREADY = 4, P_FULL = 5, P_EMPTY = 5 + MAX_RING, P_COUNT = 5 + 2 * MAX_RING };

__device__ __forceinline__ bool mbar_wait_cluster_acq(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if ((++spins & 0xFF) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
        *abort_flag = 1;
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}
__device__ __forceinline__ float4 ld_peer_f4(uint32_t local_addr, uint32_t cta) {
  uint32_t r;
  asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(cta));
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(r));
  return v;
}

__global__ void __launch_bounds__(LP_THREADS, 1)
lstm_fwd_pair_kernel(const __grid_constant__ CUtensorMap tmH, const __grid_constant__ CUtensorMap tmW, const LstmPParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int kb_half = p.kblocks / 2;
  const uint32_t w_half = p.w_bytes / 2;
  const uint32_t off_ring = (w_half + 1023u) & ~1023u;
  const uint32_t off_part = off_ring + (uint32_t)p.ring * A_STAGE;
  const uint32_t off_bar = off_part + 128u * PART_LD * 4u;
  auto bar = [&](int i) { return smem_base + off_bar + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + off_bar + 8 * P_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank(), peer = rank ^ 1u;
  const int n0 = (int)(blockIdx.x >> 1) * NC;   // first gate column of this pair
  const int kb0 = (int)rank * kb_half;          // first k-block of this CTA's half

  if (threadIdx.x == 0) {
    for (int i = 0; i < P_COUNT; i++) mbar_init(bar(i), (i == P_ACCEMPTY || i == P_STEPDONE || i == P_PARTREADY) ? 8u : 1u);   // gate warps
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(32u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  cluster_sync_all();   // the partner's barriers exist before anyone arrives on them

  if (warp == 0) {
    // ------------------------------------------------------------------ producer + grid barrier
    if (lane == 0) {
      mbar_expect_tx(bar(P_WFULL), w_half);
      for (int kb = 0; kb < kb_half; kb++) tma_load_4d(smem_base + kb * (NC * 128), &tmW, bar(P_WFULL), (kb0 + kb) * 32, n0, 0, 0);
      bool ok = true;
      uint32_t g = 0;
      for (int t = 0; t < p.T && ok; t++) {
        if (t > 0) {
          ok = mbar_wait(bar(P_STEPDONE), (uint32_t)(t - 1) & 1u, abort_flag, p.status, 51);
          if (!ok) break;
          LT_STAMP(0);
          // one release-add without a return value: the gate warps' stores of h_t (each behind its own fence, observed by this
          // thread through the mbarrier) are ordered before it, and nothing waits for the counter's old value
          asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.gbar) : "memory");
          const unsigned int target = (unsigned int)t * gridDim.x;
          const unsigned long long t0 = globaltimer_ns();
          while (ld_acquire_gpu(p.gbar) < target) {
            if (*abort_flag || globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
              *abort_flag = 1;
              atomicCAS(p.status, 0, 52);
              ok = false;
              break;
            }
          }
          if (!ok) break;
          asm volatile("fence.proxy.async.global;" ::: "memory");
          LT_STAMP(1);
        }
        for (int kb = 0; kb < kb_half && ok; kb++, g++) {
          const int s = (int)(g % (uint32_t)p.ring);
          const uint32_t ph = (g / (uint32_t)p.ring) & 1u;
          ok = mbar_wait(bar(P_EMPTY + s), ph ^ 1u, abort_flag, p.status, 53);
          if (!ok) break;
          mbar_expect_tx(bar(P_FULL + s), A_STAGE);
          tma_load_4d(smem_base + off_ring + s * A_STAGE, &tmH, bar(P_FULL + s), (kb0 + kb) * 32, t * p.B, 0, 0);
        }
        LT_STAMP(2);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(NC >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      bool ok = mbar_wait(bar(P_WFULL), 0, abort_flag, p.status, 54);
      uint32_t g = 0;
      for (int t = 0; t < p.T && ok; t++) {
        ok = mbar_wait(bar(P_ACCEMPTY), ((uint32_t)t & 1u) ^ 1u, abort_flag, p.status, 55);   // gate warps have read step t-1
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < kb_half && ok; kb++, g++) {
          const int s = (int)(g % (uint32_t)p.ring);
          const uint32_t ph = (g / (uint32_t)p.ring) & 1u;
          ok = mbar_wait(bar(P_FULL + s), ph, abort_flag, p.status, 56);
          if (!ok) break;
          if (kb == 0) LT_STAMP(3);
          tc_fence_after();
          const uint64_t ad = make_smem_desc(smem_base + off_ring + s * A_STAGE, 16u, 1024u, 2u);
          const uint64_t bd = make_smem_desc(smem_base + kb * (NC * 128), 16u, 1024u, 2u);
#pragma unroll
          for (int k = 0; k < 4; k++) umma_tf32(tmem_base, ad + 2u * k, bd + 2u * k, idesc, (kb | k) ? 1u : 0u);
          umma_commit(bar(P_EMPTY + s));
        }
        if (ok) umma_commit(bar(P_ACCFULL));
        LT_STAMP(4);
      }
    }
  } else {
    // ------------------------------------------------------------------ gate warps: thread = batch row and 2 of the CTA's 4
    // hidden units (two warps per TMEM lane quarter: the gate functions are chains of dependent special-function
    // instructions, bound by latency, so more warps shorten the phase where fewer units per thread alone did not)
    const int q4 = warp & 3;
    const int half = (warp - 2) >> 2;         // which two of the four units, and which 8 of the 16 parked columns
    const int row = q4 * 32 + lane;
    const bool active = row < p.B;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q4 * 32) << 16);
    const int N = 4 * p.H;
    const int c0 = (int)rank * 16 + half * 8;  // the 8 gate columns (of the pair's 32) this thread finalises
    const int u0 = (n0 + c0) >> 2;             // their first hidden unit
    float* part = reinterpret_cast<float*>(smem_gen + off_part);
    const uint32_t part_addr = smem_base + off_part + ((uint32_t)row * PART_LD + (uint32_t)half * 8u) * 4u;
    float c[2] = {0.f, 0.f};                   // c_0 = 0 (lstmLayer.dart:115)
    bool ok = true;
    uint32_t v[32];
    for (int t = 0; t < p.T && ok; t++) {
      float4 xa[2];
      const long long po = ((long long)t * p.B + row) * N + n0 + c0;
#pragma unroll
      for (int i = 0; i < 2; i++) xa[i] = active ? __ldg(reinterpret_cast<const float4*>(p.xproj + po) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      ok = mbar_wait_warp(bar(P_ACCFULL), (uint32_t)t & 1u, abort_flag, p.status, 57);
      if (!ok) break;
      if (threadIdx.x == 64) LT_STAMP(5);
      tc_fence_after();
      tmem_ld32(lane_addr, v);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive_warp(bar(P_ACCEMPTY));
      // park 8 of the partner's 16 columns of this CTA's partial sums, tell the partner, wait for the partner's half
      // (static register indices with selects: an index that depends on rank or warp would put the array in local memory)
      float own[8];
      {
        float* dst = part + row * PART_LD + half * 8;
#pragma unroll
        for (int i = 0; i < 8; i += 4) {
          float4 o;
          o.x = __uint_as_float(rank ? (half ? v[8 + i] : v[i]) : (half ? v[24 + i] : v[16 + i]));
          o.y = __uint_as_float(rank ? (half ? v[8 + i + 1] : v[i + 1]) : (half ? v[24 + i + 1] : v[16 + i + 1]));
          o.z = __uint_as_float(rank ? (half ? v[8 + i + 2] : v[i + 2]) : (half ? v[24 + i + 2] : v[16 + i + 2]));
          o.w = __uint_as_float(rank ? (half ? v[8 + i + 3] : v[i + 3]) : (half ? v[24 + i + 3] : v[16 + i + 3]));
          *reinterpret_cast<float4*>(dst + i) = o;
        }
#pragma unroll
        for (int i = 0; i < 8; i++) own[i] = __uint_as_float(rank ? (half ? v[24 + i] : v[16 + i]) : (half ? v[8 + i] : v[i]));
      }
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(bar(P_PARTREADY), peer);
      ok = __all_sync(0xffffffffu, mbar_wait_cluster_acq(bar(P_PARTREADY), (uint32_t)t & 1u, abort_flag, p.status, 58)) != 0;
      if (!ok) break;
      if (threadIdx.x == 64) LT_STAMP(6);
      float z[8];
#pragma unroll
      for (int i = 0; i < 8; i += 4) {
        const float4 o = ld_peer_f4(part_addr + i * 4, peer);
        z[i] = own[i] + o.x;
        z[i + 1] = own[i + 1] + o.y;
        z[i + 2] = own[i + 2] + o.z;
        z[i + 3] = own[i + 3] + o.w;
      }
      float hn[2];
      float4 gt[2];
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const float zf = z[4 * i] + xa[i].x, zi = z[4 * i + 1] + xa[i].y, zg = z[4 * i + 2] + xa[i].z, zo = z[4 * i + 3] + xa[i].w;
        float f, ig, g, o;
        if (p.fast_math) {
          f = fml_sigmoid_fast(zf); ig = fml_sigmoid_fast(zi); g = fml_tanh_fast(zg); o = fml_sigmoid_fast(zo);
        } else {
          f = fml_sigmoid(zf); ig = fml_sigmoid(zi); g = fml_tanh_ref(zg); o = fml_sigmoid(zo);
        }
        c[i] = f * c[i] + ig * g;
        hn[i] = o * (p.fast_math ? fml_tanh_fast(c[i]) : fml_tanh_ref(c[i]));
        gt[i] = make_float4(f, ig, g, o);
      }
      if (threadIdx.x == 64) LT_STAMP(7);
      const long long ho = ((long long)(t + 1) * p.B + row) * p.H + u0;
      if (active) *reinterpret_cast<float2*>(p.hs + ho) = make_float2(hn[0], hn[1]);
      __threadfence();
      asm volatile("fence.proxy.async.global;" ::: "memory");
      mbar_arrive_warp(bar(P_STEPDONE));
      if (threadIdx.x == 64) LT_STAMP(8);
      if (active) {
#pragma unroll
        for (int i = 0; i < 2; i++) reinterpret_cast<float4*>(p.gates + po)[i] = gt[i];
        *reinterpret_cast<float2*>(p.cells + ho) = make_float2(c[0], c[1]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the partner may still be reading this CTA's parked half
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32u) : "memory");
  }
}

}  // namespace

// Runs the recurrence of fml_lstm_fwd (after the input projection) in one kernel.  Returns 1 when the shape is not
// eligible (the caller falls back to the per-step kernels), 0 on success, a negative status on failure.
int32_t fml_lstm_fwd_persistent(fml_ctx* ctx, const fml_lstm_desc* d, const float* Wi, int fast_math) {
  FML_ENTER(ctx);
  const int T = d->T, B = d->B, H = d->H, I = d->I, Z = H + I;
  if (B > 128 || H % 32 != 0 || (4 * H) % NC != 0) return 1;
  const int n_cta = 4 * H / NC;
  if (n_cta > ctx->sm_count) return 1;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!al16(Wi) || !al16(d->hs) || !al16(d->xproj) || !al16(d->gates) || !al16(d->cells) || Z % 4 != 0) return 1;
  const uint32_t w_bytes = (uint32_t)NC * H * 4;
  const int kblocks = H / 32;
  const size_t fixed = ((w_bytes + 1023u) & ~1023u) + 8 * L_COUNT + 64 + 1024;
  if (fixed + 2 * A_STAGE > 220 * 1024) return 1;
  const int ring = std::min({kblocks, MAX_RING, (int)((220 * 1024 - fixed) / A_STAGE)});
  const size_t smem = fixed + (size_t)ring * A_STAGE;
  int coop = 0;
  FML_CUDA(ctx, cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx->device));
  if (!coop) return 1;

  CUtensorMap tmH, tmW;
  int32_t rc;
  // h: rows (T+1)*B of H floats; a box of 128 rows starting at t*B covers the batch (rows beyond B belong to the next
  // step or lie outside the tensor: their products are computed and ignored)
  if ((rc = fml_tc_make_tmap(ctx, d->hs, H, (int64_t)(T + 1) * B, H, 1, 1, 0, 0, 32, 128, false, 0, &tmH))) return rc;
  // Wh' = columns 0..H-1 of the gate-interleaved weight [4H x Z]
  if ((rc = fml_tc_make_tmap(ctx, Wi, H, 4 * H, Z, 1, 1, 0, 0, 32, NC, false, 0, &tmW))) return rc;
  unsigned int* gbar = nullptr;
  FML_CUDA(ctx, cudaMallocAsync(reinterpret_cast<void**>(&gbar), 256, ctx->stream));
  FML_CUDA(ctx, cudaMemsetAsync(gbar, 0, 256, ctx->stream));
  LstmPParams p;
  p.T = T; p.B = B; p.H = H; p.kblocks = kblocks; p.ring = ring; p.w_bytes = w_bytes;
  p.xproj = d->xproj; p.gates = d->gates; p.cells = d->cells; p.hs = d->hs;
  p.gbar = gbar; p.fast_math = fast_math; p.status = ctx->d_status;
  p.prof = nullptr;
#ifdef FML_LSTM_PROFILE
  static long long* prof_buf = nullptr;
  static int prof_calls = 0;
  if (!prof_buf) cudaMalloc(&prof_buf, 16 * sizeof(long long));
  p.prof = prof_buf;
#endif
  FML_ONCE_PER_DEVICE(ctx, { FML_CUDA(ctx, cudaFuncSetAttribute(lstm_fwd_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)); });
  // Two CTAs per 32 gate columns, the contraction split between them, whenever the machine holds twice the CTAs
  // (FML_LSTM_PAIR=0 keeps the one-CTA form, for comparisons).
  bool pair_done = false;
  cudaError_t e = cudaSuccess;
  {
    const char* env = getenv("FML_LSTM_PAIR");
    const size_t fixed2 = ((w_bytes / 2 + 1023u) & ~1023u) + 128 * PART_LD * 4 + 8 * P_COUNT + 64 + 1024;
    if (!(env && atoi(env) == 0) && kblocks % 2 == 0 && 2 * n_cta <= ctx->sm_count && fixed2 + 2 * A_STAGE <= 220 * 1024) {
      LstmPParams p2 = p;
      p2.ring = std::min({kblocks / 2, MAX_RING, (int)((220 * 1024 - fixed2) / A_STAGE)});
      const size_t smem2 = fixed2 + (size_t)p2.ring * A_STAGE;
      FML_ONCE_PER_DEVICE(ctx, { FML_CUDA(ctx, cudaFuncSetAttribute(lstm_fwd_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)); });
      cudaLaunchConfig_t cfg = {};
      cudaLaunchAttribute attr[2];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
      attr[1].id = cudaLaunchAttributeCooperative;
      attr[1].val.cooperative = 1;
      cfg.gridDim = dim3(2 * n_cta);
      cfg.blockDim = dim3(LP_THREADS);
      cfg.dynamicSmemBytes = smem2;
      cfg.stream = ctx->stream;
      cfg.attrs = attr;
      cfg.numAttrs = 2;
      if (cudaLaunchKernelEx(&cfg, lstm_fwd_pair_kernel, tmH, tmW, p2) == cudaSuccess) pair_done = true;
      else cudaGetLastError();   // refused: nothing ran, the one-CTA form below takes over
    }
  }
  void* args[] = {(void*)&tmH, (void*)&tmW, (void*)&p};
  if (!pair_done)
    e = cudaLaunchCooperativeKernel((void*)lstm_fwd_persistent_kernel, dim3(n_cta), dim3(LT_THREADS), args, smem, ctx->stream);
  cudaFreeAsync(gbar, ctx->stream);
#ifdef FML_LSTM_PROFILE
  if (e == cudaSuccess && ++prof_calls == 3) {
    long long h[16];
    cudaStreamSynchronize(ctx->stream);
    cudaMemcpy(h, prof_buf, sizeof h, cudaMemcpyDeviceToHost);
    fprintf(stderr, "lstm fwd, CTA 0, step 64, cycles from the moment all gate warps of the previous step had reported:\n"
                    "  grid barrier passed %lld | loads issued %lld | first h block arrived %lld | products issued %lld | accumulator ready (gate warp) %lld"
                    " | loaded %lld | gates done %lld | h stored, step reported %lld\n",
            h[1] - h[0], h[2] - h[0], h[3] - h[0], h[4] - h[0], h[5] - h[0], h[6] - h[0], h[7] - h[0], h[8] - h[0]);
  }
#endif
  if (e != cudaSuccess) {
    // the cooperative launch was refused (the grid cannot be co-resident on this device right now): nothing ran,
    // the caller takes the per-step kernels
    cudaGetLastError();
    return 1;
  }
  return FML_OK;
}
