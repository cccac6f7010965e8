// LSTM backward recurrence (BPTT): ONE cooperative kernel for all time steps (opt-in), and one fused launch per step (default).
//
// Per step the recurrence needs dh_{t-1} = dpre_t . Wh with dpre_t [B x 4H] built from dh_t, the carried dc and the
// saved gates and cells (the chain matVecMul / sigmoid / tanh / multiply backward of lib/layertypes/lstmLayer.dart:119-146
// as Tensor.backward, tensor.dart:43-75, would walk it).  As separate launches that is two dependent kernels per step
// at about 5 us of fixed cost each, more than the arithmetic.  Here the grid is (H / 128) clusters of 16 CTAs:
//   - cluster n owns 128 columns of dh; CTA r of it owns one sixteenth of the contraction (H / 4 gate columns = H / 16
//     hidden units): its slice of Wh [H/4 x 128] is loaded into shared memory once and stays there;
//   - per step the 8 compute warps (warp = 16 batch rows, lane = hidden unit, so that every global access is a
//     contiguous row segment) read dh_t, gates and cells, form the CTA's dpre tile, keep dc in REGISTERS across steps,
//     and write the tile into shared memory in the tensor core's K-major operand layout (128-byte swizzle); cluster 0
//     also stores it for the weight gradients;
//   - one thread issues the product (Wh as an MN-major B operand), every CTA copies its partial [128 x 128] from
//     tensor memory to shared memory, and each CTA sums, in a FIXED order over the sixteen CTAs (distributed shared
//     memory reads), the 8 columns it owns and stores them as dh_{t-1}: the result is reproducible, unlike the K split
//     with atomics it replaces;
//   - a grid-wide barrier (one atomic counter, bounded spin) separates the steps.
// A first version kept the A tile in tensor memory (thread = batch row): its global accesses were one 16-byte piece per
// row per instruction, 14 000 sector requests per CTA and step, and the step took 40 us.
//
// Measured (H 512, B 128, T 128, a -DFML_LSTM_PROFILE build stamps the phases of one step of CTA 0): waiting for the grid
// 10.5 us, dpre tile 5.3 us (two batches of latency-bound loads), product 0.9 us (16 instructions), copy of the partial
// tile 0.3 us, waiting for the cluster 0.9 us, the sum over sixteen CTAs through distributed shared memory 3.6 us, fence
// 0.8 us: 24 us per step, against 12 us for the two dependent launches per step it was meant to replace.  Even with the
// gate and cell loads moved in front of the grid barrier the sum over the cluster and the two barriers leave about 11 us.
// The kernel is therefore OPT-IN (FML_LSTM_BWD_SINGLE_KERNEL=1): what it offers is not speed but a recurrence whose
// result is bit for bit reproducible.  The DEFAULT is lstm_bwd_step_kernel further down: the same tiling as one launch
// per step, 7.6 us per step (0.97 ms for the 127 products of H 512, B 128, T 128).
// Every wait is bounded (mbarriers, also across the cluster: arrivals on peers' barriers instead of barrier.cluster
// inside the loop); the two cluster-wide hardware barriers, after set-up and before exit, are reached by every thread on
// every path.  Requirements: TF32 mode, batch <= 128, H a multiple of 128 and at most 512, a device that can place
// clusters of 16 CTAs; other cases use the per-step kernels.
#include <algorithm>

#include "common.cuh"
#include "tc_ptx.cuh"

int32_t fml_tc_make_tmap(fml_ctx* ctx, const float* base, int64_t cols, int64_t rows, int64_t ld, int64_t nb1, int64_t nb2,
                         int64_t s1, int64_t s2, int box_c, int box_r, bool mn_major, int blocks, CUtensorMap* out);

using namespace fml_tc;

namespace {

constexpr int KS = 16;             // CTAs per cluster = splits of the contraction
constexpr int NT = 128;            // dh columns per cluster
constexpr int LB_THREADS = 320;    // loader / grid-barrier warp, issuer warp, 8 compute warps
constexpr int PART_LD = NT + 4;    // row stride of the partial tile in shared memory (floats; the pad spreads the banks)
constexpr int ROWS_PER_WARP = 16;

struct LstmBParams {
  int T, B, H;
  int kc;                 // gate columns per CTA = 4H / KS (a multiple of 32, at most 128)
  const float* gates;     // [T][B][H][4] activated gates f, i, c~, o
  const float* cells;     // [T+1][B][H]
  float* dpre;            // [T][B][4H] gate-interleaved, written by cluster 0
  float* dh[2];           // [B][H] each; step t reads dh[t & 1] and writes dh[(t - 1) & 1]
  unsigned int* gbar;     // grid barrier counter (zeroed before the launch)
  int* status;
  unsigned long long* prof;   // -DFML_LSTM_PROFILE builds: phase time stamps of one step of CTA 0, else NULL
};

enum { B_WFULL = 0, B_AFULL = 1, B_ACCFULL = 2, B_PARTLOCAL = 3, B_PARTREADY = 4, B_STEPDONE = 5, B_GRIDOK = 6, B_COUNT = 7 };

__device__ __forceinline__ unsigned int ld_acquire_gpu_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// bounded wait with acquire semantics at cluster scope (the data it guards lives in other CTAs' shared memory)
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
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
// 16 bytes from the same shared-memory offset in CTA `cta` of the cluster.  Not volatile: the sixteen loads of a
// reduction are independent and must be in flight together (ordering comes from the barrier wait before them).
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t local_addr, uint32_t cta) {
  uint32_t r;
  asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(cta));
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(r));
  return v;
}

__global__ void __launch_bounds__(LB_THREADS, 1)
lstm_bwd_persistent_kernel(const __grid_constant__ CUtensorMap tmW, const LstmBParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t w_bytes = (uint32_t)p.kc * NT * 4;                   // Wh slice: kc/32 chunks of 32 rows x 128 columns
  const uint32_t off_a = w_bytes;                                     // A tile: kc/32 k-blocks of 128 rows x 128 bytes
  const uint32_t off_part = off_a + (uint32_t)(p.kc / 32) * 16384u;   // [128][PART_LD] floats
  const uint32_t off_bar = off_part + 128u * PART_LD * 4u;
  auto bar = [&](int i) { return smem_base + off_bar + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + off_bar + 8 * B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* part = reinterpret_cast<float*>(smem_gen + off_part);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t r = cluster_ctarank();            // which sixteenth of the contraction
  const int n = blockIdx.x / KS;                   // which 128 columns of dh
  const int G = 4 * p.H;
  const int k0 = (int)r * p.kc;                    // first gate column of this CTA
  const int products = p.T - 1;                    // steps t = T-1 .. 1 have a product; step 0 only forms dpre_0

  if (threadIdx.x == 0) {
    mbar_init(bar(B_WFULL), 1);
    mbar_init(bar(B_AFULL), 256);
    mbar_init(bar(B_ACCFULL), 1);
    mbar_init(bar(B_PARTLOCAL), 256);
    mbar_init(bar(B_PARTREADY), KS);
    mbar_init(bar(B_STEPDONE), 256);
    mbar_init(bar(B_GRIDOK), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(128u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  cluster_sync_all();   // every peer's barriers exist before anyone arrives on them remotely

  if (warp == 0) {
    // ------------------------------------------------------------------ weights once, then the step hand-overs
    if (lane == 0) {
      mbar_expect_tx(bar(B_WFULL), w_bytes);
      for (int c = 0; c < p.kc / 32; c++) tma_load_5d(smem_base + c * (32 * NT * 4), &tmW, bar(B_WFULL), 0, k0 + 32 * c, n * (NT / 32), 0, 0);
      bool ok = true;
      for (int s = 0; s < products && ok; s++) {
        // every compute thread has copied its part of the partial tile: tell the whole cluster (ourselves included)
        ok = mbar_wait(bar(B_PARTLOCAL), (uint32_t)s & 1u, abort_flag, p.status, 61);
        if (!ok) break;
        for (uint32_t c = 0; c < KS; c++) mbar_arrive_remote(bar(B_PARTREADY), c);
        // every compute thread has stored its dh_{t-1} columns: grid barrier, then release the next step
        ok = mbar_wait(bar(B_STEPDONE), (uint32_t)s & 1u, abort_flag, p.status, 62);
        if (!ok) break;
        __threadfence();
        atomicAdd(p.gbar, 1u);
        const unsigned int target = (unsigned int)(s + 1) * gridDim.x;
        const unsigned long long t0 = globaltimer_ns();
        while (ld_acquire_gpu_u32(p.gbar) < target) {
          if (*abort_flag || globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
            *abort_flag = 1;
            atomicCAS(p.status, 0, 63);
            ok = false;
            break;
          }
        }
        if (!ok) break;
        mbar_arrive(bar(B_GRIDOK));
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (0u << 15) | (1u << 16) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      bool ok = mbar_wait(bar(B_WFULL), 0, abort_flag, p.status, 64);
      for (int s = 0; s < products && ok; s++) {
        ok = mbar_wait(bar(B_AFULL), (uint32_t)s & 1u, abort_flag, p.status, 65);
        if (!ok) break;
        tc_fence_after();
        for (int c = 0; c < p.kc / 32; c++) {
          const uint64_t ad = make_smem_desc(smem_base + off_a + c * 16384, 16u, 1024u, 2u);
          const uint64_t bd = make_smem_desc(smem_base + c * (32 * NT * 4), 4096u, 512u, 1u);
#pragma unroll
          for (int k = 0; k < 4; k++) umma_tf32(tmem_base, ad + 2u * k, bd + 64u * k, idesc, (c | k) ? 1u : 0u);
        }
        umma_commit(bar(B_ACCFULL));
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    const int cw = warp - 2;                        // 0..7
    const int nuc = p.kc >> 2;                      // hidden units of this CTA (32 at H = 512)
    const bool unit_ok = lane < nuc;
    const int u = (k0 >> 2) + lane;                 // this lane's hidden unit
    // for the copy of the accumulator and the reduction: thread = (row, half), as tcgen05.ld hands rows to lanes
    const int q4 = warp & 3, half = cw >> 2;
    const int row = q4 * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q4 * 32) << 16);
    float dc[ROWS_PER_WARP];
#pragma unroll
    for (int i = 0; i < ROWS_PER_WARP; i++) dc[i] = 0.f;
    const long long bh = (long long)p.B * p.H;
    uint8_t* a_tile = smem_gen + off_a + (lane >> 3) * 16384;   // k-block of this lane's unit (8 units = 32 columns each)
    const int chunk = lane & 7;                                  // 16-byte chunk of the unit inside its k-block row
    bool ok = true;
    uint32_t v[32];
    for (int s = 0; s < p.T && ok; s++) {
      const int t = p.T - 1 - s;
#ifdef FML_LSTM_PROFILE
      const bool prof = p.prof && blockIdx.x == 0 && threadIdx.x == 64 && s == 5;
#define FML_STAMP(i) if (prof) p.prof[i] = globaltimer_ns()
#else
#define FML_STAMP(i)
#endif
      FML_STAMP(0);
      if (s > 0) {
        ok = mbar_wait(bar(B_GRIDOK), (uint32_t)(s - 1) & 1u, abort_flag, p.status, 66);
        if (!ok) break;
      }
      FML_STAMP(1);
      const float* dh_in = p.dh[t & 1];
      const float* cp_in = p.cells + (long long)t * bh;
      const float* cc_in = cp_in + bh;
      // dpre of rows [16 cw, 16 cw + 16) x this lane's unit, eight rows' loads in flight at a time
#pragma unroll
      for (int j0 = 0; j0 < ROWS_PER_WARP; j0 += 8) {
        float4 gt[8];
        float dhv[8], cpv[8], ccv[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const int rw = cw * ROWS_PER_WARP + j0 + j;
          const bool live = unit_ok && rw < p.B;
          const long long o = (long long)rw * p.H + u;
          gt[j] = live ? __ldg(reinterpret_cast<const float4*>(p.gates + ((long long)t * bh + o) * 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
          dhv[j] = live ? __ldcg(dh_in + o) : 0.f;   // written by other CTAs in the previous step: read past the L1
          cpv[j] = live ? __ldg(cp_in + o) : 0.f;
          ccv[j] = live ? __ldg(cc_in + o) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const int rw = cw * ROWS_PER_WARP + j0 + j;
          const float f = gt[j].x, ig = gt[j].y, g = gt[j].z, o = gt[j].w;
          const float tc = fml_tanh_ref(ccv[j]);
          const float d_o = dhv[j] * tc;
          const float dct = dc[j0 + j] + dhv[j] * o * (1.f - tc * tc);
          dc[j0 + j] = dct * f;
          const float4 dp = make_float4(dct * cpv[j] * (f * (1.f - f)), dct * g * (ig * (1.f - ig)), dct * ig * (1.f - g * g),
                                        d_o * (o * (1.f - o)));
          if (unit_ok) {
            if (t > 0) *reinterpret_cast<float4*>(a_tile + rw * 128 + ((chunk ^ (rw & 7)) << 4)) = dp;   // rows >= B: zeros
            if (n == 0 && rw < p.B) *reinterpret_cast<float4*>(p.dpre + ((long long)t * p.B + rw) * G + k0 + lane * 4) = dp;
          }
        }
      }
      if (t == 0) break;   // dpre_0 is formed and stored; there is no dh_{-1}
      FML_STAMP(2);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic stores of the A tile -> tensor core reads
      mbar_arrive(bar(B_AFULL));
      // the CTA's partial product [128 x 128] -> shared memory (this thread: its row, 64 columns)
      ok = mbar_wait(bar(B_ACCFULL), (uint32_t)s & 1u, abort_flag, p.status, 67);
      if (!ok) break;
      FML_STAMP(3);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; c++) {
        tmem_ld32(lane_addr + half * 64 + c * 32, v);
        tmem_ld_wait();
        float* dst = part + row * PART_LD + half * 64 + c * 32;
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          *reinterpret_cast<float4*>(dst + i) = make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]), __uint_as_float(v[i + 2]),
                                                            __uint_as_float(v[i + 3]));
      }
      tc_fence_before();   // the accumulator has been read before the next step's product overwrites it
      FML_STAMP(4);
      mbar_arrive(bar(B_PARTLOCAL));
      // all sixteen partial tiles of the cluster are in shared memory: sum the 8 columns this CTA owns, fixed order
      ok = mbar_wait_cluster(bar(B_PARTREADY), (uint32_t)s & 1u, abort_flag, p.status, 68);
      if (!ok) break;
      FML_STAMP(5);
      const int col = (int)r * (NT / KS) + half * 4;
      const uint32_t src = smem_u32(part + row * PART_LD + col);
      float4 x[KS];
#pragma unroll
      for (uint32_t c = 0; c < KS; c++) x[c] = ld_dsmem_f4(src, c);
      float4 acc = x[0];
#pragma unroll
      for (uint32_t c = 1; c < KS; c++) { acc.x += x[c].x; acc.y += x[c].y; acc.z += x[c].z; acc.w += x[c].w; }
      if (row < p.B) *reinterpret_cast<float4*>(p.dh[(t - 1) & 1] + (long long)row * p.H + n * NT + col) = acc;
      FML_STAMP(6);
      __threadfence();
      FML_STAMP(7);
      mbar_arrive(bar(B_STEPDONE));
    }
  }
  // No CTA may leave while a peer can still read its shared memory.  Reached by every thread on every path: all loops
  // above are bounded by T and by the bounded waits.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(128u) : "memory");
  }
}


// ---------------------------------------------------------------------------------------------------------------------
// One time step of the backward recurrence as ONE launch: dpre_t from dh_t, dc and the saved gates and cells, and
// dh_{t-1} = dpre_t . Wh, with the launches of consecutive steps chained by programmatic dependent launch.
//   - grid = (H / 128) column blocks x 16 slices of the contraction, as above; every CTA forms the dpre tile of ITS slice
//     itself (lane = hidden unit, warp = 16 batch rows), so no launch separates the gate derivatives from the product;
//   - everything that does not depend on the previous step is done BEFORE griddepcontrol.wait, while the previous step
//     still runs on other SMs: barriers, tensor memory, the Wh slice (a bulk tensor copy) and the saved gates and cells
//     of all sixteen rows of a thread (registers);
//   - after the wait: dh_t and dc (L2), the dpre tile into shared memory in the tensor core's operand layout, sixteen
//     MMAs, the partial [128 x 128] copied from tensor memory into a swizzled staging tile, and four bulk tensor
//     REDUCE-ADD copies into dh_{t-1}: the memory system sums the sixteen slices, whole 128-byte lines at a time;
//   - dh rotates through THREE buffers: step t reads buffer t % 3, adds into (t - 1) % 3 and zeroes (t + 1) % 3 (the
//     target of step t - 1, last read by step t + 1, which has completed when this step's wait returns).
// The sums of the slices arrive in no fixed order (as with the K-split product this replaces).
// Measured with time stamps in CTA 0 (H 512, B 128, T 128; the stamps are not kept in the source): a launch is resident
// and set up 12 us before its predecessor ends, so set-up, the weight copy and the 3.8 us of saved-state loads are hidden;
// after the wait returns (1.2 us after the predecessor's CTA 0 left: grid completion and its flush) dh and dc arrive and
// the dpre tile is in shared memory after 2.9 us (the slowest warp's L2 round trips; 1.9 us for the fastest), the
// product takes 0.9 us, the copy to the staging tile 0.4 us, the reduce-add copies until performed 1.5 us: 7.0 us from
// step to step (8.2 us per step for the whole backward pass, which also forms the weight gradients), against 12.2 us for
// the gate kernel and the K-split product as two launches.  Storing dpre and dc AFTER the hand-over to the product, and
// sharing those stores among the column blocks, did not shorten the step (7.4 us): the hand-over waits for the slowest
// warp's loads either way.  Sixteen compute warps instead of eight (eight rows per thread instead of sixteen) did: 7.0
// -> 6.4 us from step to step.  Threads that own a row x FOUR units (16-byte loads of dh, dc and the cells, four times fewer
// requests after the wait) were slower, 8.0 us: lane = hidden unit with 4-byte loads stays.
constexpr int LS_WARPS = 16;                       // compute warps: 8 batch rows each in the dpre phase, one 32-column box each in the epilogue
constexpr int LS_ROWS = 128 / LS_WARPS;
constexpr int LS_THREADS = 32 * (2 + LS_WARPS);    // + weight copy / zeroing warp, issuer warp

struct LstmStepParams {
  int B, H, kc;
  const float* gates;     // [B][H][4] of this step
  const float* c_prev;    // [B][H] cells before this step
  const float* c_cur;     // [B][H] cells after this step
  const float* dh_in;     // [B][H]
  const float* dc_in;     // [B][H]
  float* dc_out;          // [B][H], written by column block 0
  float* dh_zero;         // [B][H] the buffer the NEXT launch accumulates into
  float* dpre;            // [B][4H] of this step, written by column block 0
  int* status;
};

enum { S_WFULL = 0, S_AFULL = 1, S_ACCFULL = 2, S_COUNT = 3 };

__global__ void __launch_bounds__(LS_THREADS, 1)
lstm_bwd_step_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmDH, const LstmStepParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t w_bytes = (uint32_t)p.kc * NT * 4;     // Wh slice: kc/32 chunks of 32 rows x 128 columns
  const uint32_t off_a = w_bytes;                       // A tile (kc/32 k-blocks of 16 KB), then reused as the staging tile (64 KB)
  const uint32_t off_bar = off_a + 65536u;
  auto bar = [&](int i) { return smem_base + off_bar + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + off_bar + 8 * S_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x % KS;                   // which sixteenth of the contraction
  const int n = blockIdx.x / KS;                   // which 128 columns of dh
  const int G = 4 * p.H;
  const int k0 = r * p.kc;                         // first gate column of this CTA

  if (threadIdx.x == 0) {
    mbar_init(bar(S_WFULL), 1);
    mbar_init(bar(S_AFULL), LS_WARPS);
    mbar_init(bar(S_ACCFULL), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(128u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // the next step's launch may begin its own set-up on the idle SMs from here on
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      // the weights do not depend on the previous step
      mbar_expect_tx(bar(S_WFULL), w_bytes);
      for (int c = 0; c < p.kc / 32; c++) tma_load_5d(smem_base + c * (32 * NT * 4), &tmW, bar(S_WFULL), 0, k0 + 32 * c, n * (NT / 32), 0, 0);
    }
    // this warp zeroes the CTA's share of the buffer the next launch adds into (a buffer the previous launch read)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int n4 = (p.B * p.H) >> 2;
    float4* z = reinterpret_cast<float4*>(p.dh_zero);
    for (int i = blockIdx.x * 32 + lane; i < n4; i += gridDim.x * 32) z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (0u << 15) | (1u << 16) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      bool ok = mbar_wait(bar(S_WFULL), 0, abort_flag, p.status, 71);
      ok = ok && mbar_wait(bar(S_AFULL), 0, abort_flag, p.status, 72);
      if (ok) {
        tc_fence_after();
        for (int c = 0; c < p.kc / 32; c++) {
          const uint64_t ad = make_smem_desc(smem_base + off_a + c * 16384, 16u, 1024u, 2u);
          const uint64_t bd = make_smem_desc(smem_base + c * (32 * NT * 4), 4096u, 512u, 1u);
#pragma unroll
          for (int k = 0; k < 4; k++) umma_tf32(tmem_base, ad + 2u * k, bd + 64u * k, idesc, (c | k) ? 1u : 0u);
        }
        umma_commit(bar(S_ACCFULL));
      }
    }
  } else {
    const int cw = warp - 2;                        // 0..15
    const int nuc = p.kc >> 2;                      // hidden units of this CTA (32 at H = 512)
    const bool unit_ok = lane < nuc;
    const int u = (k0 >> 2) + lane;                 // this lane's hidden unit
    uint8_t* a_tile = smem_gen + off_a + (lane >> 3) * 16384;   // k-block of this lane's unit (8 units = 32 columns each)
    const int chunk = lane & 7;                                  // 16-byte chunk of the unit inside its k-block row
    // saved state of this thread's eight (row, unit) elements: independent of the previous step
    float4 gt[LS_ROWS];
    float cpv[LS_ROWS], ccv[LS_ROWS];
#pragma unroll
    for (int j = 0; j < LS_ROWS; j++) {
      const int rw = cw * LS_ROWS + j;
      const bool live = unit_ok && rw < p.B;
      const long long o = (long long)rw * p.H + u;
      gt[j] = live ? __ldg(reinterpret_cast<const float4*>(p.gates) + o) : make_float4(0.f, 0.f, 0.f, 0.f);
      cpv[j] = live ? __ldg(p.c_prev + o) : 0.f;
      ccv[j] = live ? __ldg(p.c_cur + o) : 0.f;
    }
    // tanh of the cell does not depend on the previous step either
#pragma unroll
    for (int j = 0; j < LS_ROWS; j++) ccv[j] = fml_tanh_ref(ccv[j]);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float dhv[LS_ROWS], dcv[LS_ROWS];
#pragma unroll
    for (int j = 0; j < LS_ROWS; j++) {
      const int rw = cw * LS_ROWS + j;
      const bool live = unit_ok && rw < p.B;
      const long long o = (long long)rw * p.H + u;
      dhv[j] = live ? __ldcg(p.dh_in + o) : 0.f;   // summed by the previous launch in L2
      dcv[j] = live ? __ldcg(p.dc_in + o) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < LS_ROWS; j++) {
      const int rw = cw * LS_ROWS + j;
      const float f = gt[j].x, ig = gt[j].y, g = gt[j].z, o = gt[j].w;
      const float tc = ccv[j];
      const float d_o = dhv[j] * tc;
      const float dct = dcv[j] + dhv[j] * o * (1.f - tc * tc);
      const float4 dp = make_float4(dct * cpv[j] * (f * (1.f - f)), dct * g * (ig * (1.f - ig)), dct * ig * (1.f - g * g),
                                    d_o * (o * (1.f - o)));
      if (unit_ok) {
        *reinterpret_cast<float4*>(a_tile + rw * 128 + ((chunk ^ (rw & 7)) << 4)) = dp;   // rows >= B: zeros
        if (n == 0 && rw < p.B) {
          *reinterpret_cast<float4*>(p.dpre + (long long)rw * G + k0 + lane * 4) = dp;
          p.dc_out[(long long)rw * p.H + u] = dct * f;
        }
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic stores of the A tile -> tensor core reads
    mbar_arrive_warp(bar(S_AFULL));
    // the partial product [128 x 128] -> staging tile (four boxes of 32 columns, 128-byte swizzle) -> reduce-add into dh
    const int q4 = warp & 3, box = cw >> 2;          // tcgen05.ld hands lanes 32 q4 .. 32 q4 + 31 to warp % 4 == q4
    const int row = q4 * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q4 * 32) << 16);
    const bool ok = mbar_wait_warp(bar(S_ACCFULL), 0, abort_flag, p.status, 73);
    if (ok) {
      tc_fence_after();
      uint32_t v[32];
      tmem_ld32(lane_addr + box * 32, v);
      tmem_ld_wait();
      uint8_t* dst = smem_gen + off_a + box * 16384 + row * 128;
#pragma unroll
      for (int i = 0; i < 8; i++)
        *reinterpret_cast<float4*>(dst + ((i ^ (row & 7)) << 4)) =
            make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]), __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    asm volatile("bar.sync 1, %0;" ::"n"(32 * LS_WARPS) : "memory");   // the compute warps; reached on every path
    if (ok && threadIdx.x == 64) {
#pragma unroll
      for (int b = 0; b < 4; b++) tma_reduce_add_4d(&tmDH, smem_base + off_a + b * 16384, n * NT + b * 32, 0, 0, 0);
      tma_store_commit();
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // performed, not only read: the next launch reads the sums
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(128u) : "memory");
  }
}

}  // namespace

// Runs the recurrence of fml_lstm_bwd (dpre of every step and the dh chain) in one kernel.  dh_a and dh_b are two
// [B x H] buffers; dh_last is copied into the one step T-1 reads.  Returns 1 when the shape is not eligible or the
// cooperative cluster launch is refused (the caller falls back to the per-step kernels), 0 on success, a negative status
// on failure.
int32_t fml_lstm_bwd_persistent(fml_ctx* ctx, const fml_lstm_desc* d, const float* Wi, const float* dh_last, float* dpre,
                                float* dh_a, float* dh_b) {
  FML_ENTER(ctx);
  const int T = d->T, B = d->B, H = d->H, I = d->I, Z = H + I;
  if (B > 128 || H % NT != 0 || H > 512 || T < 1) return 1;
  const int kc = 4 * H / KS;
  if (kc % 32 != 0 || kc > 128) return 1;
  const int n_cta = (H / NT) * KS;
  if (n_cta > ctx->sm_count) return 1;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!al16(Wi) || !al16(d->gates) || !al16(d->cells) || !al16(dpre) || !al16(dh_a) || !al16(dh_b) || Z % 4 != 0) return 1;
  int coop = 0;
  FML_CUDA(ctx, cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx->device));
  if (!coop) return 1;
  const size_t smem = (size_t)kc * NT * 4 + (size_t)(kc / 32) * 16384 + (size_t)128 * PART_LD * 4 + 8 * B_COUNT + 64 + 1024;
  if (smem > 227 * 1024) return 1;

  CUtensorMap tmW;
  int32_t rc;
  // Wh = columns 0..H-1 of the gate-interleaved weight [4H x Z]: rows are the contraction (gate columns), columns the
  // dh columns, so it is an MN-major B operand: boxes of 32 rows x 4 blocks of 32 columns
  if ((rc = fml_tc_make_tmap(ctx, Wi, H, 4 * H, Z, 1, 1, 0, 0, 32, 32, true, NT / 32, &tmW))) return rc;
  float* dh[2] = {dh_a, dh_b};
  FML_CUDA(ctx, cudaMemcpyAsync(dh[(T - 1) & 1], dh_last, (size_t)B * H * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  unsigned int* gbar = nullptr;
  FML_CUDA(ctx, cudaMallocAsync(reinterpret_cast<void**>(&gbar), 256, ctx->stream));
  FML_CUDA(ctx, cudaMemsetAsync(gbar, 0, 256, ctx->stream));
  LstmBParams p;
  p.T = T; p.B = B; p.H = H; p.kc = kc;
  p.gates = d->gates; p.cells = d->cells; p.dpre = dpre;
  p.dh[0] = dh[0]; p.dh[1] = dh[1];
  p.gbar = gbar; p.status = ctx->d_status;
  p.prof = nullptr;
#ifdef FML_LSTM_PROFILE
  static unsigned long long* prof_buf = nullptr;
  if (!prof_buf) cudaMalloc(&prof_buf, 64);
  p.prof = prof_buf;
#endif
  FML_ONCE_PER_DEVICE(ctx, {
    FML_CUDA(ctx, cudaFuncSetAttribute(lstm_bwd_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    // clusters of 16 CTAs are beyond the portable size of 8: the device has to allow them (B200 does)
    if (cudaFuncSetAttribute(lstm_bwd_persistent_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
      cudaGetLastError();
      cudaFreeAsync(gbar, ctx->stream);
      return 1;
    }
  });
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = KS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeCooperative;
  attr[1].val.cooperative = 1;
  cfg.gridDim = dim3(n_cta);
  cfg.blockDim = dim3(LB_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaError_t e = cudaLaunchKernelEx(&cfg, lstm_bwd_persistent_kernel, tmW, p);
  cudaFreeAsync(gbar, ctx->stream);
#ifdef FML_LSTM_PROFILE
  if (e == cudaSuccess) {
    unsigned long long h[8];
    cudaStreamSynchronize(ctx->stream);
    cudaMemcpy(h, p.prof, sizeof h, cudaMemcpyDeviceToHost);
    fprintf(stderr, "lstm bwd, CTA 0, step 5 (ns): grid wait %llu | dpre %llu | product %llu | copy partial %llu | cluster wait %llu | reduce+store %llu | fence %llu\n",
            h[1] - h[0], h[2] - h[1], h[3] - h[2], h[4] - h[3], h[5] - h[4], h[6] - h[5], h[7] - h[6]);
  }
#endif
  if (e != cudaSuccess) {
    // refused (the clusters cannot all be co-resident right now, or the combination is not supported): nothing ran
    cudaGetLastError();
    return 1;
  }
  return FML_OK;
}

// The recurrence of fml_lstm_bwd as one launch per time step (lstm_bwd_step_kernel), steps T-1 .. 1; the caller forms
// dpre_0 from the returned buffers.  work holds five [B x H] buffers (three for dh, two for dc).  On success *dh_final
// and *dc_final are the buffers holding dh_0 and the dc flowing into step 0.  Returns 1 when the shape is not eligible.
int32_t fml_lstm_bwd_steps(fml_ctx* ctx, const fml_lstm_desc* d, const float* Wi, const float* dh_last, float* dpre, float* work,
                           float** dh_final, float** dc_final) {
  FML_ENTER(ctx);
  const int T = d->T, B = d->B, H = d->H, I = d->I, Z = H + I;
  if (B > 128 || H % NT != 0 || H > 512 || T < 1) return 1;
  const int kc = 4 * H / KS;
  if (kc % 32 != 0 || kc > 128) return 1;
  const int n_cta = (H / NT) * KS;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!al16(Wi) || !al16(d->gates) || !al16(d->cells) || !al16(dpre) || !al16(work) || Z % 4 != 0) return 1;
  const size_t smem = (size_t)kc * NT * 4 + 65536 + 8 * S_COUNT + 64 + 1024;
  const long long bh = (long long)B * H, b4h = 4 * bh;
  float* dh[3] = {work, work + bh, work + 2 * bh};
  float* dc[2] = {work + 3 * bh, work + 4 * bh};
  CUtensorMap tmW, tmDH[3];
  int32_t rc;
  if ((rc = fml_tc_make_tmap(ctx, Wi, H, 4 * H, Z, 1, 1, 0, 0, 32, 32, true, NT / 32, &tmW))) return rc;
  for (int i = 0; i < 3; i++)
    if ((rc = fml_tc_make_tmap(ctx, dh[i], H, B, H, 1, 1, 0, 0, 32, 128, false, 0, &tmDH[i]))) return rc;
  FML_ONCE_PER_DEVICE(ctx, {
    FML_CUDA(ctx, cudaFuncSetAttribute(lstm_bwd_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
  });
  FML_CUDA(ctx, cudaMemsetAsync(work, 0, (size_t)5 * bh * 4, ctx->stream));
  FML_CUDA(ctx, cudaMemcpyAsync(dh[(T - 1) % 3], dh_last, (size_t)bh * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  for (int t = T - 1; t >= 1; t--) {
    LstmStepParams p;
    p.B = B; p.H = H; p.kc = kc;
    p.gates = d->gates + t * b4h;
    p.c_prev = d->cells + t * bh;
    p.c_cur = d->cells + (t + 1) * bh;
    p.dh_in = dh[t % 3];
    p.dh_zero = dh[(t + 1) % 3];
    p.dc_in = dc[t & 1];
    p.dc_out = dc[(t - 1) & 1];
    p.dpre = dpre + t * b4h;
    p.status = ctx->d_status;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3(n_cta);
    cfg.blockDim = dim3(LS_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    FML_CUDA(ctx, cudaLaunchKernelEx(&cfg, lstm_bwd_step_kernel, tmW, tmDH[(t - 1) % 3], p));
  }
  *dh_final = dh[0];
  *dc_final = dc[0];
  return FML_OK;
}
