// Fused scaled-dot-product attention forward on the tensor cores: for one block of 128 queries of one
// (sequence, head) the kernel walks the key/value blocks.  S = Q.K^T lands in tensor memory, sixteen softmax warps turn
// it into probabilities IN PLACE (tcgen05.ld -> registers -> tcgen05.st over the same columns; scale and causal mask
// folded in, base-2 exponentials), and the second product P.V reads its A operand straight from tensor memory and
// accumulates the output in tensor memory across all key blocks.  Neither the scores nor the probabilities touch
// shared or global memory: the reference's transpose + matMul + scaleMatrix + softmaxMatrix + matMul chain
// (lib/layertypes/singleHeadAttentionLayer.dart:77-86) becomes one pass over Q, K, V.
//
// One CTA = 640 threads:
//   warp 0      TMA producer: Q and K_j (two-stage ring); when all loads of an item are issued it prefetches the next
//               item's Q into L2
//   warp 1      MMA issuer: S_j = Q.K_j^T into one of two TMEM buffers (S_{j+1} is issued before P_j.V_j, so it runs
//               under the softmax of block j), then O += P_j.V_j once the softmax warps have published P_j
//   warps 2..17 softmax: thread = one query row (TMEM lane) and a quarter of the block's keys, 32 scores in registers
//               (four warps per lane quarter, so that every scheduler has four warps to choose from).  The exponent
//               reference m of a row is only moved when a block's maximum exceeds it by more than 2^8; until then the
//               probabilities are formed against the old reference (they stay below 2^8, the row sum carries the same
//               factor), so the accumulator in tensor memory needs no rescaling and the warps never wait for P.V.
//               The output pass of an item is deferred behind the first softmax of the next item.
//   warp 18     TMA producer of V_j (three-stage ring)
//   warp 19     stores: the normalised output tile goes through a 16 KiB staging tile, half by half, with tile stores
// Shared memory: Q, 2 x K, 3 x V of 32 KiB, 8 KiB row exchange, 16 KiB output staging.  TMEM: S/P buffers [0,128) and [128,256), two O
// accumulators [256,320) and [320,384) that alternate from item to item.
// V is consumed as an MN-major B operand (32-byte-atom swizzle, the layout notes of gemm_tc.cu apply).
// Requirements: d_head = 64, seq_len a multiple of 128, 16-byte aligned rows.  Every mbarrier wait is bounded.
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "tc_ptx.cuh"

int32_t fml_tc_make_tmap(fml_ctx* ctx, const float* base, int64_t cols, int64_t rows, int64_t ld, int64_t nb1, int64_t nb2,
                         int64_t s1, int64_t s2, int box_c, int box_r, bool mn_major, int blocks, CUtensorMap* out);

using namespace fml_tc;

namespace {

constexpr int BQ = 128, BKV = 128, DH = 64;
constexpr int FA_THREADS = 640;      // forward: Q/K producer, issuer, 16 softmax warps (four per TMEM lane quarter, 32 keys each), V producer, store warp
constexpr int FA_BWD_THREADS = 352;  // dQ kernel: producer, issuer, 8 compute warps (two per TMEM lane quarter, alternate 32-column chunks), store warp
constexpr int FA_DKV_THREADS = 608;  // dK/dV kernel: producer, issuer, 16 compute warps (four per TMEM lane quarter, one 32-query chunk each), store warp
constexpr uint32_t OFF_Q = 0, OFF_K = 32768, OFF_V = 98304, OFF_XCH = 196608, OFF_ST = 204800, OFF_BAR = 229376;   // forward: Q, 2 x K, 3 x V, row exchange, output staging (16 KiB)
constexpr int FA_SMEM = OFF_BAR + 256 + 2048 + 512;   // barriers, the row exchange (forward), alignment slack
constexpr int K_STAGES = 2, V_STAGES = 3;   // a V tile arrived about 5000 cycles after its buffer came free (measured): two stages stalled every item's first P.V
constexpr uint32_t TM_S = 0, TM_O = 256;   // two S/P buffers of 128 columns, two O accumulators of 64 columns (alternate items)
constexpr int FA_MAX_SEQ_TMEM_P = 512;    // longest sequence the tensor-memory forward kernel is used for (four key blocks per item)
constexpr float FA_RESCALE_LOG2 = 8.f;   // a row's exponent reference moves only when a block maximum exceeds it by 2^8

struct FaParams {
  int S, H, n_qb;        // sequence length, heads, query blocks per sequence
  int n_items;           // n_seq * H * n_qb work items
  int round_p;           // 1: P is rounded to TF32 before it is summed and multiplied (0 only for diagnostics, FML_FA_NOROUND)
  int causal;
  float k2;              // scale * log2(e)
  float* out; long long ld_out;
  float* lse;            // [n_seq][H][S]: m + log2(l) of every row in the scaled base-2 domain, or NULL
  int* status;
  long long* prof;       // -DFML_FA_PROFILE builds: clock64 stamps of key blocks 8..15 of CTA 0, else NULL
};

// Phase stamps for the diagnostics build (-DFML_FA_PROFILE): slot k of key block g, blocks 8..15 of CTA 0 only.
#ifdef FML_FA_PROFILE
#define FA_STAMP(prof, g, k) do { if ((prof) && blockIdx.x == 0 && (g) >= 8u && (g) < 16u) (prof)[((g) - 8u) * 16u + (k)] = clock64(); } while (0)
#define FA_TOTAL_BEGIN() const long long fa_c0 = clock64(); const unsigned long long fa_n0 = globaltimer_ns()
#define FA_TOTAL_END(prof) do { if ((prof) && threadIdx.x == 0) { (prof)[128 + 2 * blockIdx.x] = clock64() - fa_c0; (prof)[129 + 2 * blockIdx.x] = (long long)(globaltimer_ns() - fa_n0); } } while (0)
#else
#define FA_STAMP(prof, g, k) do { } while (0)
#define FA_TOTAL_BEGIN() do { } while (0)
#define FA_TOTAL_END(prof) do { } while (0)
#endif

// barriers: Q full/empty, K ring full/empty, V ring full/empty, S full (per buffer), P full (per buffer), P.V done (per
// buffer), O read by the softmax warps
enum { B_QFULL = 0, B_QEMPTY = 1, B_KFULL = 2, B_KEMPTY = 4, B_VFULL = 6, B_VEMPTY = 9, B_SFULL = 12, B_PFULL = 14, B_PVDONE = 16,
       B_OEMPTY = 18 /* one per O accumulator */, B_ROW = 20 /* one per lane quarter: the four threads of a row meet here */, B_STAGED = 24, B_STFREE = 25 /* one per half of the output tile */, B_COUNT = 27 };

// 2^x on the special-function unit with flush-to-zero: the library exp2f adds a rescaling sequence for results below
// 2^-126, which are zero for every purpose here
__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Round-to-nearest (ties away from zero) of a finite float to TF32 (10 mantissa bits) with two integer instructions;
// the sign bit rides along.  The tensor core itself TRUNCATES fp32 operands to TF32 (measured: a product of operands
// cut to 19 bits on the host reproduces the device result to 3e-7, and products of generic data come out 7.0e-4 low,
// 3.5e-4 per operand).  Every operand this file builds on chip (P, dS and their transposes) is therefore rounded here
// first, which removes that operand's share of the bias; Q, K, V, dO arrive by TMA and are used as they are.
__device__ __forceinline__ float fa_round_tf32(float x) { return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u); }
__device__ __forceinline__ uint32_t fa_idesc(int M, int N, int a_mn, int b_mn) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(a_mn & 1) << 15) | ((uint32_t)(b_mn & 1) << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__global__ void __launch_bounds__(FA_THREADS, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const FaParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  auto bar = [&](int i) { return smem_base + OFF_BAR + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + OFF_BAR + 8 * B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The layout leaves 512 bytes of slack for rounding the dynamic shared memory base up to 1 KiB.  Should a driver ever
  // hand out a base that needs more, every thread leaves here (same condition for all) and the host reads code 7.
  if ((smem_base - smem_u32(smem_raw)) + OFF_BAR + 256u > (uint32_t)FA_SMEM) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, 7);
    return;
  }

  // Persistent loop: this CTA takes work items blockIdx.x, blockIdx.x + gridDim.x, ...  Items are ordered heaviest
  // first (all last query blocks, then the ones before, ...), so the causal triangle spreads evenly over the CTAs.
  // Barrier phases are driven by running counters (g = key blocks processed so far, it = items), which lets the
  // producer and the MMA issuer run ahead into the next item while the softmax warps finish the current one.
  const int n_bh = p.n_items / p.n_qb;
  auto item_coords = [&](int item, int& qb, int& h, int& b, int& n_kv) {
    // CTAs walk the item list in alternating directions from round to round (full rounds only), which evens out the block
    // counts: with plain striding CTA c gets the same rank in every round and the heaviest CTAs end 4 % above the mean.
    {
      const int G = gridDim.x, k = item / G;
      if ((k & 1) && k < p.n_items / G) item = k * G + (G - 1 - (item - k * G));
    }
    qb = p.n_qb - 1 - item / n_bh;
    const int bh = item - (item / n_bh) * n_bh;
    h = bh % p.H;
    b = bh / p.H;
    n_kv = p.causal ? qb + 1 : p.S / BKV;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < B_COUNT; i++) {
      const bool from_softmax = (i == B_PFULL || i == B_PFULL + 1 || i == B_OEMPTY || i == B_OEMPTY + 1);
      mbar_init(bar(i), from_softmax ? 16u : (i == B_STAGED ? 8u : (i >= B_STFREE ? 1u : (i >= B_ROW ? 4u : 1u))));   // warps, not threads (mbar_arrive_warp)
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  FA_TOTAL_BEGIN();

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      bool ok = true;
      uint32_t g = 0, it = 0;
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, it++) {
        int qb, h, b, n_kv;
        item_coords(item, qb, h, b, n_kv);
        // Q is single-buffered (the previous item's last S product must have read it); it was prefetched into L2
        ok = mbar_wait(bar(B_QEMPTY), (it & 1u) ^ 1u, abort_flag, p.status, 10);
        if (!ok) break;
        mbar_expect_tx(bar(B_QFULL), BQ * DH * 4);
        for (int kb = 0; kb < 2; kb++) tma_load_4d(smem_base + OFF_Q + kb * 16384, &tmQ, bar(B_QFULL), kb * 32, qb * BQ, h, b);
        for (int j = 0; j < n_kv && ok; j++, g++) {
          const int s = g % K_STAGES;
          const uint32_t ph = (g / K_STAGES) & 1u;
          ok = mbar_wait(bar(B_KEMPTY + s), ph ^ 1u, abort_flag, p.status, 11);
          if (!ok) break;
          mbar_expect_tx(bar(B_KFULL + s), BKV * DH * 4);
          for (int kb = 0; kb < 2; kb++)
            tma_load_4d(smem_base + OFF_K + s * 32768 + kb * 16384, &tmK, bar(B_KFULL + s), kb * 32, j * BKV, h, b);
        }
        if (ok && item + (int)gridDim.x < p.n_items) {
          // Q of the next item into L2: its load is issued only when this item's last S product has read the buffer, one
          // block before it is needed, and from DRAM it took about 4000 cycles under load (measured)
          int qb2, h2, b2, n2;
          item_coords(item + gridDim.x, qb2, h2, b2, n2);
          for (int kb = 0; kb < 2; kb++) tma_prefetch_4d(&tmQ, kb * 32, qb2 * BQ, h2, b2);
        }
      }
    }
  } else if (warp == 18) {
    // ------------------------------------------------------------------ V producer (its own thread: a V buffer comes free
    // one P.V product later than the K buffer of the same block, and one thread loading both held the K loads back)
    if (lane == 0) {
      bool ok = true;
      uint32_t g = 0;
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x) {
        int qb, h, b, n_kv;
        item_coords(item, qb, h, b, n_kv);
        for (int j = 0; j < n_kv && ok; j++, g++) {
          const int s = g % V_STAGES;
          const uint32_t ph = (g / V_STAGES) & 1u;
          ok = mbar_wait(bar(B_VEMPTY + s), ph ^ 1u, abort_flag, p.status, 9);
          if (!ok) break;
          mbar_expect_tx(bar(B_VFULL + s), BKV * DH * 4);
          for (int c = 0; c < 4; c++)
            tma_load_5d(smem_base + OFF_V + s * 32768 + c * 8192, &tmV, bar(B_VFULL + s), 0, j * BKV + 32 * c, 0, h, b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = fa_idesc(BQ, BKV, 0, 0), idesc_pv = fa_idesc(BQ, DH, 0, 1);
      bool ok = true;
      // Cursor of the next S product: it runs one key block ahead of the P.V products, across item boundaries.  S_{g+1}
      // overwrites the TMEM buffer P_{g-1} lived in; P_{g-1}.V_{g-1} was issued earlier by this thread and tensor-core
      // operations execute in issue order, so no barrier is needed for that hand-over.
      int s_item = blockIdx.x, s_j = 0, s_nkv = 0;
      uint32_t s_g = 0, s_it = 0;
      if (s_item < p.n_items) { int a, b2, c; item_coords(s_item, a, b2, c, s_nkv); }
      auto issue_next_s = [&]() {
        if (s_item >= p.n_items) return true;
        const int ks = s_g % K_STAGES;
        const uint32_t kph = (s_g / K_STAGES) & 1u;
        const int buf = s_g & 1;
        if (s_j == 0 && !mbar_wait(bar(B_QFULL), s_it & 1u, abort_flag, p.status, 12)) return false;
        if (!mbar_wait(bar(B_KFULL + ks), kph, abort_flag, p.status, 13)) return false;
        FA_STAMP(p.prof, s_g - 1u, 14);   // operands of the next S product ready
        tc_fence_after();
        for (int kb = 0; kb < 2; kb++) {
          const uint64_t ad = make_smem_desc(smem_base + OFF_Q + kb * 16384, 16u, 1024u, 2u);
          const uint64_t bd = make_smem_desc(smem_base + OFF_K + ks * 32768 + kb * 16384, 16u, 1024u, 2u);
#pragma unroll
          for (int k = 0; k < 4; k++) umma_tf32(tmem_base + TM_S + buf * 128, ad + 2u * k, bd + 2u * k, idesc_s, (kb | k) ? 1u : 0u);
        }
        umma_commit(bar(B_SFULL + buf));
        umma_commit(bar(B_KEMPTY + ks));   // K_j is read by nothing else
        s_g++;
        if (++s_j == s_nkv) {   // last S of its item: Q may be replaced
          umma_commit(bar(B_QEMPTY));
          s_item += gridDim.x;
          s_it++;
          s_j = 0;
          if (s_item < p.n_items) { int a, b2, c; item_coords(s_item, a, b2, c, s_nkv); }
        }
        return true;
      };
      uint32_t g = 0, it = 0;
      ok = issue_next_s();
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, it++) {
        int qb, h, b, n_kv;
        item_coords(item, qb, h, b, n_kv);
        for (int j = 0; j < n_kv && ok; j++, g++) {
          const int vs = g % V_STAGES;
          const uint32_t vph = (g / V_STAGES) & 1u;
          const int buf = g & 1;
          FA_STAMP(p.prof, g, 8);
          if (s_g == g + 1) ok = issue_next_s();   // keep one S product ahead
          if (!ok) break;
          FA_STAMP(p.prof, g, 9);
          // the first P.V of an item overwrites its O accumulator (items alternate between two): the softmax warps must
          // have read the output of the item before the previous one
          if (j == 0) ok = mbar_wait(bar(B_OEMPTY + (it & 1u)), ((it >> 1) & 1u) ^ 1u, abort_flag, p.status, 8);
          FA_STAMP(p.prof, g, 12);
          ok = ok && mbar_wait(bar(B_PFULL + buf), (g >> 1) & 1u, abort_flag, p.status, 15);
          FA_STAMP(p.prof, g, 15);
          ok = ok && mbar_wait(bar(B_VFULL + vs), vph, abort_flag, p.status, 16);
          if (!ok) break;
          FA_STAMP(p.prof, g, 10);
          tc_fence_after();
          for (int c = 0; c < 4; c++) {  // 32 keys per chunk of V, 8 keys per instruction
            const uint64_t bd = make_smem_desc(smem_base + OFF_V + vs * 32768 + c * 8192, 4096u, 512u, 1u);
#pragma unroll
            for (int k = 0; k < 4; k++)
              umma_tf32_ts(tmem_base + TM_O + (it & 1u) * 64, tmem_base + TM_S + buf * 128 + c * 32 + k * 8, bd + 64u * k, idesc_pv, (j | c | k) ? 1u : 0u);
          }
          umma_commit(bar(B_PVDONE + buf));
          umma_commit(bar(B_VEMPTY + vs));
          FA_STAMP(p.prof, g, 11);
          if (j == n_kv - 1) FA_STAMP(p.prof, g, 13);   // slot 13 is written on the last block of an item only
        }
      }
    }
  } else if (warp == 19) {
    // ------------------------------------------------------------------ store warp: the output tile of every finished item
    // leaves in two halves of 32 columns through one 16 KiB staging tile.  Stored row by row from the registers it cost
    // 16 warps x 4 instructions x 32 separate lines, and while the load/store unit worked through them the issuer's
    // barrier polls queued behind (measured: 1700 cycles between an operand being ready and the issuer noticing).
    if (lane == 0) {
      bool ok = true;
      uint32_t n = 0;
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x) {
        int qb, h, b, n_kv;
        item_coords(item, qb, h, b, n_kv);
        for (int r = 0; r < 2 && ok; r++, n++) {
          ok = mbar_wait(bar(B_STAGED), n & 1u, abort_flag, p.status, 48);
          if (!ok) break;
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          tma_store_4d(&tmO, smem_base + OFF_ST, r * 32, qb * BQ, h, b);
          tma_store_commit();
          tma_store_wait_read();
          mbar_arrive(bar(B_STFREE + r));
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / output
    // Four warps per TMEM lane quarter: thread = one query row and one QUARTER of the block's 128 keys (32 scores in
    // registers).  The four threads of a row agree on the block maximum through shared memory (two 128-thread named
    // barriers per block); everything else (probabilities, partial row sum, the thread's 16 output columns) needs no
    // exchange.  Sixteen softmax warps give every scheduler four warps to choose from: with one or two, the issue slots
    // stayed three quarters empty (tensor-memory loads, the exponential's latency and the barriers all stall a warp).
    const int q4 = warp & 3;                        // TMEM lane quarter of this warp
    const int part = (warp - 2) >> 2;               // which 32 keys of every block, and which 16 output columns
    const int row = q4 * 32 + lane;                 // row inside the query block
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q4 * 32) << 16);
    // Row exchange, [2][4 parts][128 rows] of {block maximum, share of the finished item's row sum}: the buffers alternate
    // from block to block, so one meeting per block is enough (a thread can be at most one meeting ahead of its
    // partners, and then writes the other buffer), and the row sum of a finished item rides along with the first
    // maximum of the next one instead of costing two more meetings.
    float2* xch = reinterpret_cast<float2*>(smem_gen + OFF_XCH);
    // The meeting point of a row's four threads is an mbarrier, not a named hardware barrier: its wait is bounded like
    // every other wait of this kernel, so a CTA that gives up somewhere cannot leave partner warps parked forever.
    uint32_t n_sync = 0;
    auto row_sync = [&]() {
      mbar_arrive_warp(bar(B_ROW + q4));
      return mbar_wait_warp(bar(B_ROW + q4), (n_sync++) & 1u, abort_flag, p.status, 5);
    };
    bool ok = true;
    uint32_t v0[32];
    uint32_t o16[16];
    uint32_t g = 0;
    // The output pass of a finished item (wait for its last P.V, normalise, store) is deferred until the first block of the
    // NEXT item has been turned into probabilities: done right away it kept the tensor pipe idle for the whole pass plus
    // that block's softmax (measured: 6000 cycles per item against 2400 per key block).
    bool pending = false;
    float pend_m = 0.f, pend_l = 0.f, pend_lt = 0.f;   // exponent reference, this thread's share of the row sum, the row sum
    long long pend_stat = 0;
    uint32_t pend_g = 0, pend_o = 0, it = 0, n_out = 0;
    auto finish_item = [&]() {   // pend_lt is known by now
      if (!mbar_wait_warp(bar(B_PVDONE + (pend_g & 1)), (pend_g >> 1) & 1u, abort_flag, p.status, 19)) return false;
      tc_fence_after();
      tmem_ld16(lane_addr + TM_O + pend_o * 64 + part * 16, o16);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive_warp(bar(B_OEMPTY + pend_o));   // this accumulator may be overwritten by the item after the next
      const float inv = 1.f / pend_lt;
      // parts 0, 1 fill the staging tile with columns [0,32), parts 2, 3 with [32,64) once the first half has been read
      // Two barriers, one per half: a parity wait can only tell the current phase from the previous one, so every waiter
      // must see every phase of its barrier, in order.  Parts 0, 1 wait for the previous item's second half to have been
      // read, parts 2, 3 for this item's first half.  (With one barrier for both, a thread that looked at every other
      // phase overwrote a half that had not been read yet whenever a tile store took longer than a key block.)
      if (part < 2) {
        if (!mbar_wait_warp(bar(B_STFREE + 1), (n_out & 1u) ^ 1u, abort_flag, p.status, 49)) return false;
      } else {
        if (!mbar_wait_warp(bar(B_STFREE), n_out & 1u, abort_flag, p.status, 50)) return false;
      }
      uint8_t* srow = smem_gen + OFF_ST + row * 128;   // 128-byte rows, 16-byte chunks swizzled (the tile store's layout)
#pragma unroll
      for (int i = 0; i < 4; i++)
        *reinterpret_cast<float4*>(srow + ((((part & 1) * 4 + i) ^ (row & 7)) << 4)) =
            make_float4(__uint_as_float(o16[4 * i]) * inv, __uint_as_float(o16[4 * i + 1]) * inv, __uint_as_float(o16[4 * i + 2]) * inv,
                        __uint_as_float(o16[4 * i + 3]) * inv);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive_warp(bar(B_STAGED));
      n_out++;
      if (p.lse && part == 0) p.lse[pend_stat] = pend_m + log2f(pend_lt);
#ifdef FML_FA_PROFILE
      if (threadIdx.x == 64) FA_STAMP(p.prof, pend_g, 7);   // end of the item's output pass
#endif
      pending = false;
      return true;
    };
    for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x) {
      int qb, h, b, n_kv;
      item_coords(item, qb, h, b, n_kv);
      const int qi = qb * BQ + row;                 // position in the sequence
      float m = -INFINITY, l = 0.f;                 // l: this thread's share of the row sum
      for (int j = 0; j < n_kv && ok; j++, g++) {
        const int buf = g & 1;
        const uint32_t sp = lane_addr + TM_S + buf * 128 + part * 32;
#ifdef FML_FA_PROFILE
        long long* const sprof = threadIdx.x == 64 ? p.prof : nullptr;
#else
        long long* const sprof = nullptr;
        (void)sprof;
#endif
        FA_STAMP(sprof, g, 0);
#ifdef FML_FA_PROFILE
        if (p.prof && blockIdx.x == 0 && lane == 0 && g == 12u) p.prof[464 + warp] = clock64();   // every warp's arrival at the item's first block
#endif
        ok = mbar_wait_warp(bar(B_SFULL + buf), (g >> 1) & 1u, abort_flag, p.status, 17);
        if (!ok) break;
        FA_STAMP(sprof, g, 1);
        tc_fence_after();
        tmem_ld32(sp, v0);
        tmem_ld_wait();
        FA_STAMP(sprof, g, 2);
        const bool diag = p.causal && j == qb;
        const int lim = (diag ? row + 1 : BKV) - part * 32;   // valid keys of this row inside this thread's part
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (diag) {
#pragma unroll
          for (int e = 0; e < 32; e++) mx4[e & 3] = fmaxf(mx4[e & 3], (e < lim) ? __uint_as_float(v0[e]) : -INFINITY);
        } else {
#pragma unroll
          for (int e = 0; e < 32; e++) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(v0[e]));
        }
        float2* xb = xch + (g & 1u) * 512;
        xb[part * 128 + row] = make_float2(fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])), pend_l);
        ok = row_sync();
        if (!ok) break;
        FA_STAMP(sprof, g, 3);
        const float2 e0 = xb[row], e1 = xb[128 + row], e2 = xb[256 + row], e3 = xb[384 + row];
        const float bm = fmaxf(fmaxf(e0.x, e1.x), fmaxf(e2.x, e3.x)) * p.k2;   // k2 > 0
        if (pending) pend_lt = (e0.y + e1.y) + (e2.y + e3.y);
        FA_STAMP(sprof, g, 4);
        // Move the reference where a block maximum exceeds it by 2^8 (the four threads of a row take the same decision from
        // the same numbers).  Block 0 of an item always moves it (m = -inf) with nothing to rescale; in later blocks the
        // accumulator in tensor memory is rescaled, which the previous P.V must have finished writing.  The tensor-memory
        // accesses are warp-wide instructions, so the whole warp goes through them as soon as one of its rows moves; rows that
        // keep their reference scale by one.
        const bool move = bm > m + FA_RESCALE_LOG2;
        if (j > 0 && __any_sync(0xffffffffu, move)) {
          ok = mbar_wait_warp(bar(B_PVDONE + (buf ^ 1)), ((g - 1) >> 1) & 1u, abort_flag, p.status, 18);
          if (!ok) break;
          tc_fence_after();
          const float alpha = move ? fa_exp2(m - bm) : 1.f;
          tmem_ld16(lane_addr + TM_O + (it & 1u) * 64 + part * 16, o16);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; e++) o16[e] = __float_as_uint(__uint_as_float(o16[e]) * alpha);
          tmem_st16(lane_addr + TM_O + (it & 1u) * 64 + part * 16, o16);
          l *= alpha;
        }
        if (move) m = bm;
        // probabilities (unnormalised, below 2^8) over the scores, rounded to TF32; the ROUNDED value enters the row sum:
        // the tensor core would otherwise cut the low mantissa bits of P on its own and bias every output low
        float ls4[4] = {0.f, 0.f, 0.f, 0.f};
        const float k2 = p.k2, nm = -m;
        const bool rnd = p.round_p != 0;
#pragma unroll
        for (int e = 0; e < 32; e++) {
          float p0 = fa_exp2(fmaf(__uint_as_float(v0[e]), k2, nm));
          if (rnd) p0 = fa_round_tf32(p0);
          if (diag) p0 = (e < lim) ? p0 : 0.f;
          ls4[e & 3] += p0;
          v0[e] = __float_as_uint(p0);
        }
        l += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
        FA_STAMP(sprof, g, 5);
        tmem_st32(sp, v0);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive_warp(bar(B_PFULL + buf));
        FA_STAMP(sprof, g, 6);
#ifdef FML_FA_PROFILE
        if (p.prof && blockIdx.x == 0 && lane == 0 && (g == 12u || g == 13u)) p.prof[424 + (g - 12u) * 20 + warp] = clock64();   // every warp's publish time
#endif
        if (pending) {   // the previous item's output, now that this item's first P.V has its operand
          ok = finish_item();
          if (!ok) break;
        }
      }
      if (ok) {
        pending = true;
        pend_m = m;
        pend_l = l;
        pend_stat = ((long long)b * p.H + h) * p.S + qi;
        pend_g = g - 1;
        pend_o = it & 1u;
      }
      it++;
    }
    if (ok && pending) {   // the CTA's last item: no next block to ride along with
      float2* xb = xch + (g & 1u) * 512;
      xb[part * 128 + row] = make_float2(0.f, pend_l);
      ok = row_sync();
      if (ok) {
        pend_lt = (xb[row].y + xb[128 + row].y) + (xb[256 + row].y + xb[384 + row].y);
        ok = finish_item();
      }
    }
  }
  FA_TOTAL_END(p.prof);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------------------
// Forward for sequences longer than 512: the same products with the probabilities staged through shared memory (a
// K-major A operand with a hand-written 128-byte swizzle) and the output accumulated in registers, one softmax warp per
// lane quarter.  It is the slower of the two forward kernels per key block, and the one whose long-sequence behaviour
// has been verified (up to 8 x 16 x 2048, many work items per CTA); the kernel above is used where IT has been
// verified, i.e. for up to four key blocks per work item.
// Shared memory (224 KiB): Q 32 KiB, 2 x K 32 KiB, 2 x V 32 KiB, P 64 KiB.  TMEM: S0 [0,128), S1 [128,256), PV [256,320).
constexpr int FA_LONG_THREADS = 192;   // producer, issuer, 4 softmax warps
constexpr uint32_t LO_Q = 0, LO_K = 32768, LO_V = 98304, LO_P = 163840;
constexpr uint32_t LT_S = 0, LT_PV = 256;
enum { L_QFULL = 0, L_KFULL = 1, L_VFULL = 3, L_KVEMPTY = 5, L_SFULL = 7, L_SEMPTY = 9, L_PFULL = 11, L_PVFULL = 12, L_QEMPTY = 13, L_COUNT = 14 };

__global__ void __launch_bounds__(FA_LONG_THREADS, 1)
attention_fwd_long_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const FaParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  auto bar = [&](int i) { return smem_base + OFF_BAR + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + OFF_BAR + 8 * L_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Persistent loop: this CTA takes work items blockIdx.x, blockIdx.x + gridDim.x, ...  Items are ordered heaviest
  // first (all last query blocks, then the ones before, ...), so the causal triangle spreads evenly over the CTAs.
  // Barrier phases are driven by running counters (g = key blocks processed so far, it = items), which lets the
  // producer and the MMA issuer run ahead into the next item while the softmax warps finish the current one.
  const int n_bh = p.n_items / p.n_qb;
  auto item_coords = [&](int item, int& qb, int& h, int& b, int& n_kv) {
    qb = p.n_qb - 1 - item / n_bh;
    const int bh = item - (item / n_bh) * n_bh;
    h = bh % p.H;
    b = bh / p.H;
    n_kv = p.causal ? qb + 1 : p.S / BKV;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < L_COUNT; i++) {
      const bool from_softmax = (i == L_SEMPTY || i == L_SEMPTY + 1 || i == L_PFULL);
      mbar_init(bar(i), from_softmax ? 128u : 1u);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      bool ok = true;
      uint32_t g = 0, it = 0;
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, it++) {
        int qb, h, b, n_kv;
        item_coords(item, qb, h, b, n_kv);
        // Q is single-buffered: the previous item's last S product must have read it
        ok = mbar_wait(bar(L_QEMPTY), (it & 1u) ^ 1u, abort_flag, p.status, 10);
        if (!ok) break;
        mbar_expect_tx(bar(L_QFULL), BQ * DH * 4);
        for (int kb = 0; kb < 2; kb++) tma_load_4d(smem_base + LO_Q + kb * 16384, &tmQ, bar(L_QFULL), kb * 32, qb * BQ, h, b);
        for (int j = 0; j < n_kv && ok; j++, g++) {
          const int s = g & 1;
          const uint32_t ph = (g >> 1) & 1u;
          ok = mbar_wait(bar(L_KVEMPTY + s), ph ^ 1u, abort_flag, p.status, 11);
          if (!ok) break;
          mbar_expect_tx(bar(L_KFULL + s), BKV * DH * 4);
          for (int kb = 0; kb < 2; kb++)
            tma_load_4d(smem_base + LO_K + s * 32768 + kb * 16384, &tmK, bar(L_KFULL + s), kb * 32, j * BKV, h, b);
          mbar_expect_tx(bar(L_VFULL + s), BKV * DH * 4);
          for (int c = 0; c < 4; c++)
            tma_load_5d(smem_base + LO_V + s * 32768 + c * 8192, &tmV, bar(L_VFULL + s), 0, j * BKV + 32 * c, 0, h, b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = fa_idesc(BQ, BKV, 0, 0), idesc_pv = fa_idesc(BQ, DH, 0, 1);
      bool ok = true;
      // cursor of the next S product to issue: it runs one key block ahead of the P.V products, across item boundaries
      int s_item = blockIdx.x, s_j = 0, s_nkv = 0;
      uint32_t s_g = 0, s_it = 0;
      if (s_item < p.n_items) { int a, b2, c; item_coords(s_item, a, b2, c, s_nkv); }
      auto issue_next_s = [&]() {
        if (s_item >= p.n_items) return true;
        const int s = s_g & 1;
        const uint32_t ph = (s_g >> 1) & 1u;
        if (s_j == 0 && !mbar_wait(bar(L_QFULL), s_it & 1u, abort_flag, p.status, 12)) return false;
        if (!mbar_wait(bar(L_KFULL + s), ph, abort_flag, p.status, 13)) return false;
        if (!mbar_wait(bar(L_SEMPTY + s), ph ^ 1u, abort_flag, p.status, 14)) return false;
        tc_fence_after();
        for (int kb = 0; kb < 2; kb++) {
          const uint64_t ad = make_smem_desc(smem_base + LO_Q + kb * 16384, 16u, 1024u, 2u);
          const uint64_t bd = make_smem_desc(smem_base + LO_K + s * 32768 + kb * 16384, 16u, 1024u, 2u);
#pragma unroll
          for (int k = 0; k < 4; k++) umma_tf32(tmem_base + LT_S + s * 128, ad + 2u * k, bd + 2u * k, idesc_s, (kb | k) ? 1u : 0u);
        }
        umma_commit(bar(L_SFULL + s));
        s_g++;
        if (++s_j == s_nkv) {   // last S of its item: Q may be replaced
          umma_commit(bar(L_QEMPTY));
          s_item += gridDim.x;
          s_it++;
          s_j = 0;
          if (s_item < p.n_items) { int a, b2, c; item_coords(s_item, a, b2, c, s_nkv); }
        }
        return true;
      };
      uint32_t g = 0;
      ok = issue_next_s();
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x) {
        int qb, h, b, n_kv;
        item_coords(item, qb, h, b, n_kv);
        for (int j = 0; j < n_kv && ok; j++, g++) {
          const int s = g & 1;
          const uint32_t ph = (g >> 1) & 1u;
          if (s_g == g + 1) ok = issue_next_s();   // keep one S product ahead
          if (!ok) break;
          ok = mbar_wait(bar(L_PFULL), g & 1u, abort_flag, p.status, 15) && mbar_wait(bar(L_VFULL + s), ph, abort_flag, p.status, 16);
          if (!ok) break;
          tc_fence_after();
          for (int c = 0; c < 4; c++) {  // 32 keys per chunk
            const uint64_t ad = make_smem_desc(smem_base + LO_P + c * 16384, 16u, 1024u, 2u);
            const uint64_t bd = make_smem_desc(smem_base + LO_V + s * 32768 + c * 8192, 4096u, 512u, 1u);
#pragma unroll
            for (int k = 0; k < 4; k++) umma_tf32(tmem_base + LT_PV, ad + 2u * k, bd + 64u * k, idesc_pv, (c | k) ? 1u : 0u);
          }
          umma_commit(bar(L_PVFULL));       // PV readable, P free again
          umma_commit(bar(L_KVEMPTY + s));  // K and V of this block consumed
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / output
    const int q4 = warp & 3;                        // TMEM lane quarter of this warp
    const int row = q4 * 32 + lane;                 // row inside the query block
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q4 * 32) << 16);
    bool ok = true;
    uint32_t v[32];
    uint32_t g = 0;
    for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x) {
      int qb, h, b, n_kv;
      item_coords(item, qb, h, b, n_kv);
      const int qi = qb * BQ + row;                 // position in the sequence
      float m = -INFINITY, l = 0.f;
      float o[DH];
#pragma unroll
      for (int i = 0; i < DH; i++) o[i] = 0.f;
      for (int j = 0; j < n_kv && ok; j++, g++) {
        const int s = g & 1;
        ok = mbar_wait(bar(L_SFULL + s), (g >> 1) & 1u, abort_flag, p.status, 17);
        if (!ok) break;
        tc_fence_after();
        const bool diag = p.causal && j == qb;
        const int lim = diag ? row + 1 : BKV;        // valid keys of this row inside the block
        // pass 1: row maximum of the scores (four chains instead of one of 128 dependent maxima)
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        for (int c = 0; c < 4; c++) {
          tmem_ld32(lane_addr + LT_S + s * 128 + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; e++) {
            const float sc = (c * 32 + e < lim) ? __uint_as_float(v[e]) : -INFINITY;
            mx4[e & 3] = fmaxf(mx4[e & 3], sc);
          }
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.k2;   // k2 > 0: max commutes with the scale
        const float m_new = fmaxf(m, mx);            // finite: key 0 is visible to every row
        const float alpha = fa_exp2(m - m_new);        // 0 for the first block (m = -inf)
        // the previous block's P.V must be folded in (and P be free) before P is overwritten
        if (j > 0) {
          ok = mbar_wait(bar(L_PVFULL), (g - 1) & 1u, abort_flag, p.status, 18);
          if (!ok) break;
          tc_fence_after();
          for (int c = 0; c < 2; c++) {
            tmem_ld32(lane_addr + LT_PV + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; e++) o[c * 32 + e] += __uint_as_float(v[e]);
          }
        }
#pragma unroll
        for (int i = 0; i < DH; i++) o[i] *= alpha;
        l *= alpha;
        // pass 2: probabilities (unnormalised) into the K-major operand layout: k-block c = 32 keys = one 128-byte row
        // per query, 16-byte chunks XOR-swizzled with the row index
        float ls4[4] = {0.f, 0.f, 0.f, 0.f};
        for (int c = 0; c < 4; c++) {
          tmem_ld32(lane_addr + LT_S + s * 128 + c * 32, v);
          tmem_ld_wait();
          uint8_t* prow = smem_gen + LO_P + c * 16384 + row * 128;
#pragma unroll
          for (int ch = 0; ch < 8; ch++) {
            float4 pv;
            float* pe = reinterpret_cast<float*>(&pv);
#pragma unroll
            for (int e = 0; e < 4; e++) {
              const int col = c * 32 + ch * 4 + e;
              // rounded to TF32 here, and the ROUNDED value enters the row sum: the tensor core would otherwise cut the
              // low mantissa bits of P on its own and every output would come out low by up to 2^-11 relative to l
              const float pe_ = fa_exp2(fmaf(__uint_as_float(v[ch * 4 + e]), p.k2, -m_new));
              const float pr = (col < lim) ? (p.round_p ? fa_round_tf32(pe_) : pe_) : 0.f;
              pe[e] = pr;
              ls4[e] += pr;
            }
            *reinterpret_cast<float4*>(prow + ((ch ^ (row & 7)) << 4)) = pv;
          }
        }
        l += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
        m = m_new;
        tc_fence_before();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(bar(L_PFULL));
        mbar_arrive(bar(L_SEMPTY + s));
      }
      if (ok) ok = mbar_wait(bar(L_PVFULL), (g - 1) & 1u, abort_flag, p.status, 19);
      if (ok) {
        tc_fence_after();
        for (int c = 0; c < 2; c++) {
          tmem_ld32(lane_addr + LT_PV + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; e++) o[c * 32 + e] += __uint_as_float(v[e]);
        }
        // the P.V accumulator has been read: order these loads before the next item's first P.V product
        tc_fence_before();
        const float inv = 1.f / l;
        float* orow = p.out + ((long long)b * p.S + qi) * p.ld_out + h * DH;
#pragma unroll
        for (int i = 0; i < DH; i += 4)
          *reinterpret_cast<float4*>(orow + i) = make_float4(o[i] * inv, o[i + 1] * inv, o[i + 2] * inv, o[i + 3] * inv);
        if (p.lse) p.lse[((long long)b * p.H + h) * p.S + qi] = m + log2f(l);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

}  // namespace

namespace {

// ------------------------------------------------------------------------------------------------------------
// Backward, first kernel: for one block of 128 queries it rebuilds the probabilities of every key block from the
// saved row statistics, forms dS = scale * P * (dP - D) with dP = dO.V^T and D = rowsum(dO * O), and accumulates
// dQ = dS.K over the key blocks in TMEM.  dS never leaves tensor memory: the compute warps write it over dP
// (tcgen05.st) and the third product reads its A operand from there.
//   warp 0      TMA: Q, dO; per key block K_j, V_j (K-major) and K_j again as an MN-major B operand (two buffers)
//   warp 1      MMA, in this order on the tensor pipe: ... dP_j, S_{j+1}, dQ_j, dP_{j+1}, S_{j+2}, dQ_{j+1} ...
//               S_{j+1} = Q.K_{j+1}^T is issued BEFORE the issuer waits for dS_j, so the exponentials of block j+1 run
//               under dQ_j += dS_j.K_j; dP_{j+1} = dO.V_{j+1}^T follows dQ_j because it overwrites dS_j (the pipe
//               executes in issue order, no barrier needed for that hand-over)
//   warps 2..9  thread = query row and two of the four 32-column chunks.  Phase A (needs S only): P = 2^(S k2 - L) into
//               registers.  Phase B (needs dP): dS = round_tf32(scale P (dP - D)) over dP in tensor memory.
// The running counters g (key blocks) and it (items) drive every barrier phase, so all three roles run on across item
// boundaries; the dQ tile of a finished item is read after the next item's first dS has been published, and the issuer
// holds that item's first dQ product back until every warp has read (C_DQREAD).
//   warp 10     stores: the dQ tile of a finished item goes from tensor memory through a swizzled shared-memory tile
//               to global memory with one tile store (accumulate form: a tile reduction).  Written row by row from the
//               registers (thread = row) the tile cost every warp 8 instructions x 32 separate lines, about 3000 cycles
//               of load/store-unit time per item on the critical path (measured).
// Shared memory (224 KiB): Q, dO, K, V 32 KiB each, K(MN) 2 x 32 KiB, dQ staging 32 KiB.  Q of the next item is
// prefetched into L2 (two instructions), so its load after the item's last S product is short.
// TMEM: S [0,128) and [128,256), dP/dS [256,384), dQ [384,448).
constexpr uint32_t BO_Q = 0, BO_DO = 32768, BO_K = 65536, BO_V = 98304, BO_KMN = 131072, BO_ST = 196608;
constexpr uint32_t TM_DP = 256, TM_DQ = 384;
enum { C_QFULL = 0, C_QEMPTY = 2, C_DOFULL = 4, C_DOEMPTY = 5, C_KFULL = 6, C_KEMPTY = 7, C_VFULL = 8, C_VEMPTY = 9, C_KMNFULL = 10,
       C_KMNEMPTY = 12, C_SFULL = 14, C_SEMPTY = 16, C_DPFULL = 18, C_DSFULL = 19, C_DQDONE = 20, C_STAGED = 21, C_STFREE = 22, C_DQREAD = 23, C_COUNT = 24 };

struct FaBwdParams {
  int S, H, n_qb, causal;
  int n_items;
  float k2, scale;
  const float* lse;   // [n_seq][H][S]
  const float* dsum;  // [n_seq][H][S]: D = rowsum(dO * O)
  float* dq; long long ld_dq;
  int accumulate;
  int* status;
  long long* prof;    // -DFML_FA_PROFILE builds, else NULL
};

__global__ void __launch_bounds__(FA_BWD_THREADS, 1)
attention_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                        const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                        const __grid_constant__ CUtensorMap tmKmn, const __grid_constant__ CUtensorMap tmDQ, const FaBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  auto bar = [&](int i) { return smem_base + OFF_BAR + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + OFF_BAR + 8 * C_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // persistent loop over work items (heaviest first)
  const int n_bh = p.n_items / p.n_qb;
  auto item_coords = [&](int item, int& qb, int& h, int& b, int& n_kv) {
    // CTAs walk the item list in alternating directions from round to round (full rounds only), which evens out the block
    // counts: with plain striding CTA c gets the same rank in every round and the heaviest CTAs end 4 % above the mean.
    {
      const int G = gridDim.x, k = item / G;
      if ((k & 1) && k < p.n_items / G) item = k * G + (G - 1 - (item - k * G));
    }
    qb = p.n_qb - 1 - item / n_bh;
    const int bh = item - (item / n_bh) * n_bh;
    h = bh % p.H;
    b = bh / p.H;
    n_kv = p.causal ? qb + 1 : p.S / BKV;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < C_COUNT; i++) {
      const bool from_compute = (i == C_SEMPTY || i == C_SEMPTY + 1 || i == C_DSFULL || i == C_STAGED || i == C_DQREAD);
      mbar_init(bar(i), from_compute ? 8u : 1u);   // warps, not threads (mbar_arrive_warp)
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  FA_TOTAL_BEGIN();

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      uint32_t g = 0, it = 0;
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, it++) {
        int qb, h, b, n_kv;
        item_coords(item, qb, h, b, n_kv);
        ok = mbar_wait(bar(C_QEMPTY), (it & 1u) ^ 1u, abort_flag, p.status, 20);   // the previous item's last S has read it
        if (!ok) break;
        mbar_expect_tx(bar(C_QFULL), BQ * DH * 4);
        for (int kb = 0; kb < 2; kb++) tma_load_4d(smem_base + BO_Q + kb * 16384, &tmQ, bar(C_QFULL), kb * 32, qb * BQ, h, b);
        for (int j = 0; j < n_kv && ok; j++, g++) {
          const uint32_t ph = g & 1u, ms = g & 1u;
          ok = mbar_wait(bar(C_KEMPTY), ph ^ 1u, abort_flag, p.status, 22);
          if (!ok) break;
          mbar_expect_tx(bar(C_KFULL), BKV * DH * 4);
          for (int kb = 0; kb < 2; kb++) tma_load_4d(smem_base + BO_K + kb * 16384, &tmK, bar(C_KFULL), kb * 32, j * BKV, h, b);
          ok = mbar_wait(bar(C_KMNEMPTY + ms), ((g >> 1) & 1u) ^ 1u, abort_flag, p.status, 31);
          if (!ok) break;
          mbar_expect_tx(bar(C_KMNFULL + ms), BKV * DH * 4);
          for (int c = 0; c < 4; c++)
            tma_load_5d(smem_base + BO_KMN + ms * 32768 + c * 8192, &tmKmn, bar(C_KMNFULL + ms), 0, j * BKV + 32 * c, 0, h, b);
          if (j == 0) {
            // dO after the first K of the item: the wait below ends only when the previous item's last dP has run, and the
            // next S product (which needs K, not dO) must not queue behind it
            ok = mbar_wait(bar(C_DOEMPTY), (it & 1u) ^ 1u, abort_flag, p.status, 21);
            if (!ok) break;
            mbar_expect_tx(bar(C_DOFULL), BQ * DH * 4);
            for (int kb = 0; kb < 2; kb++) tma_load_4d(smem_base + BO_DO + kb * 16384, &tmDO, bar(C_DOFULL), kb * 32, qb * BQ, h, b);
          }
          ok = mbar_wait(bar(C_VEMPTY), ph ^ 1u, abort_flag, p.status, 32);
          if (!ok) break;
          mbar_expect_tx(bar(C_VFULL), BKV * DH * 4);
          for (int kb = 0; kb < 2; kb++) tma_load_4d(smem_base + BO_V + kb * 16384, &tmV, bar(C_VFULL), kb * 32, j * BKV, h, b);
          if (j == 0 && item + (int)gridDim.x < p.n_items) {
            // Q of the next item into L2 (more prefetching was measured to cost more than it saves: a prefetch occupies
            // this SM's copy engine like a load, and the loads of the running item queue behind it)
            int qb2, h2, b2, n2;
            item_coords(item + gridDim.x, qb2, h2, b2, n2);
            for (int kb = 0; kb < 2; kb++) tma_prefetch_4d(&tmQ, kb * 32, qb2 * BQ, h2, b2);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = fa_idesc(BQ, BKV, 0, 0), idesc_dq = fa_idesc(BQ, DH, 0, 1);
      bool ok = true;
      // cursor of the next S product: one key block ahead of the dP / dQ products, across item boundaries
      int s_item = blockIdx.x, s_j = 0, s_nkv = 0;
      uint32_t s_g = 0, s_it = 0;
      if (s_item < p.n_items) { int a, b2, c; item_coords(s_item, a, b2, c, s_nkv); }
      auto issue_next_s = [&]() {
        if (s_item >= p.n_items) return true;
        const uint32_t buf = s_g & 1u;
        if (s_j == 0 && !mbar_wait(bar(C_QFULL), s_it & 1u, abort_flag, p.status, 23)) return false;
        if (!mbar_wait(bar(C_KFULL), s_g & 1u, abort_flag, p.status, 24)) return false;
        if (!mbar_wait(bar(C_SEMPTY + buf), ((s_g >> 1) & 1u) ^ 1u, abort_flag, p.status, 25)) return false;   // phase A of block s_g-2 done
        FA_STAMP(p.prof, s_g - 1u, 11);   // operands of the next S product ready
        tc_fence_after();
        for (int kb = 0; kb < 2; kb++) {
          const uint64_t aq = make_smem_desc(smem_base + BO_Q + kb * 16384, 16u, 1024u, 2u);
          const uint64_t bk = make_smem_desc(smem_base + BO_K + kb * 16384, 16u, 1024u, 2u);
#pragma unroll
          for (int k = 0; k < 4; k++) umma_tf32(tmem_base + TM_S + buf * 128, aq + 2u * k, bk + 2u * k, idesc_s, (kb | k) ? 1u : 0u);
        }
        umma_commit(bar(C_SFULL + buf));
        umma_commit(bar(C_KEMPTY));
        s_g++;
        if (++s_j == s_nkv) {   // last S of its item: Q may be replaced
          umma_commit(bar(C_QEMPTY));
          s_item += gridDim.x;
          s_it++;
          s_j = 0;
          if (s_item < p.n_items) { int a, b2, c; item_coords(s_item, a, b2, c, s_nkv); }
        }
        return true;
      };
      uint32_t g = 0, it = 0;
      ok = issue_next_s();
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, it++) {
        int qb, h, b, n_kv;
        item_coords(item, qb, h, b, n_kv);
        for (int j = 0; j < n_kv && ok; j++, g++) {
          const uint32_t ph = g & 1u, ms = g & 1u;
          // dP_g: overwrites dS_{g-1}, which dQ_{g-1} (issued earlier by this thread) has read by then
          FA_STAMP(p.prof, g, 8);
          if (j == 0) ok = mbar_wait(bar(C_DOFULL), it & 1u, abort_flag, p.status, 26);
          ok = ok && mbar_wait(bar(C_VFULL), ph, abort_flag, p.status, 27);
          if (!ok) break;
          FA_STAMP(p.prof, g, 9);
          tc_fence_after();
          for (int kb = 0; kb < 2; kb++) {
            const uint64_t ad = make_smem_desc(smem_base + BO_DO + kb * 16384, 16u, 1024u, 2u);
            const uint64_t bv = make_smem_desc(smem_base + BO_V + kb * 16384, 16u, 1024u, 2u);
#pragma unroll
            for (int k = 0; k < 4; k++) umma_tf32(tmem_base + TM_DP, ad + 2u * k, bv + 2u * k, idesc_s, (kb | k) ? 1u : 0u);
          }
          umma_commit(bar(C_DPFULL));
          umma_commit(bar(C_VEMPTY));
          if (j == n_kv - 1) umma_commit(bar(C_DOEMPTY));
          FA_STAMP(p.prof, g, 10);
          if (s_g == g + 1) ok = issue_next_s();   // S_{g+1} runs under the compute phase of block g
          if (!ok) break;
          FA_STAMP(p.prof, g, 12);
          ok = mbar_wait(bar(C_DSFULL), ph, abort_flag, p.status, 28) && mbar_wait(bar(C_KMNFULL + ms), (g >> 1) & 1u, abort_flag, p.status, 29);
          // the first dQ product of an item overwrites the accumulator: the compute warps must have read the previous item's
          if (ok && j == 0 && it > 0) ok = mbar_wait(bar(C_DQREAD), (it - 1) & 1u, abort_flag, p.status, 54);
          if (!ok) break;
          FA_STAMP(p.prof, g, 13);
          tc_fence_after();
          for (int c = 0; c < 4; c++) {   // 32 keys per chunk of K, 8 keys per instruction, A operand = dS in tensor memory
            const uint64_t bd = make_smem_desc(smem_base + BO_KMN + ms * 32768 + c * 8192, 4096u, 512u, 1u);
#pragma unroll
            for (int k = 0; k < 4; k++)
              umma_tf32_ts(tmem_base + TM_DQ, tmem_base + TM_DP + c * 32 + k * 8, bd + 64u * k, idesc_dq, (j | c | k) ? 1u : 0u);
          }
          umma_commit(bar(C_DQDONE));
          umma_commit(bar(C_KMNEMPTY + ms));
          FA_STAMP(p.prof, g, 14);
          if (j == n_kv - 1) FA_STAMP(p.prof, g, 15);   // slot 15 on the last block of an item only
        }
      }
    }
  } else if (warp == FA_BWD_THREADS / 32 - 1) {
    // ------------------------------------------------------------------ store warp
    if (lane == 0) {
      bool ok = true;
      uint32_t it = 0;
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, it++) {
        int qb, h, b, n_kv;
        item_coords(item, qb, h, b, n_kv);
        ok = mbar_wait(bar(C_STAGED), it & 1u, abort_flag, p.status, 48);   // all 256 rows of the tile are in shared memory
        if (!ok) break;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        for (int kb = 0; kb < 2; kb++) {
          if (p.accumulate) tma_reduce_add_4d(&tmDQ, smem_base + BO_ST + kb * 16384, kb * 32, qb * BQ, h, b);
          else tma_store_4d(&tmDQ, smem_base + BO_ST + kb * 16384, kb * 32, qb * BQ, h, b);
        }
        tma_store_commit();
        tma_store_wait_read();            // the staging tile has been read: the next item may overwrite it
        mbar_arrive(bar(C_STFREE));
      }
    }
  } else {
    const int q4 = warp & 3;
    const int half = (warp - 2) >> 2;   // the two warps of a lane quarter take alternate 32-column chunks
    const int row = q4 * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q4 * 32) << 16);
    bool ok = true;
    uint32_t tv[32];
    float pr[64];
    uint32_t g = 0, n_flush = 0;
    bool pending = false;        // a finished item whose dQ tile is still to be read
    auto flush_dq = [&]() {      // after dQ of block g-1 (the pending item's last) has been accumulated
      if (!mbar_wait_warp(bar(C_DQDONE), (g - 1) & 1u, abort_flag, p.status, 30)) return false;
      tc_fence_after();
      tmem_ld32(lane_addr + TM_DQ + half * 32, tv);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive_warp(bar(C_DQREAD));   // the issuer holds the next item's first dQ product back until all warps are here
      if (!mbar_wait_warp(bar(C_STFREE), (n_flush & 1u) ^ 1u, abort_flag, p.status, 49)) return false;   // previous tile stored
      uint8_t* srow = smem_gen + BO_ST + half * 16384 + row * 128;   // K-major tile layout: 128-byte rows, 16-byte chunks swizzled
#pragma unroll
      for (int ch = 0; ch < 8; ch++)
        *reinterpret_cast<float4*>(srow + ((ch ^ (row & 7)) << 4)) =
            make_float4(__uint_as_float(tv[4 * ch]), __uint_as_float(tv[4 * ch + 1]), __uint_as_float(tv[4 * ch + 2]), __uint_as_float(tv[4 * ch + 3]));
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive_warp(bar(C_STAGED));
      n_flush++;
      pending = false;
      return true;
    };
    // The row statistics of an item are loaded one item ahead: read at the item's start they cost a DRAM round trip
    // (2000 cycles, measured) in front of its first exponentials.
    float L_next = 0.f, D_next = 0.f;
    auto load_stats = [&](int item) {
      if (item >= p.n_items) return;
      int qb, h, b, n_kv;
      item_coords(item, qb, h, b, n_kv);
      const long long stat = ((long long)b * p.H + h) * p.S + qb * BQ + row;
      L_next = __ldg(p.lse + stat);
      D_next = __ldg(p.dsum + stat);
    };
    load_stats(blockIdx.x);
    for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x) {
      int qb, h, b, n_kv;
      item_coords(item, qb, h, b, n_kv);
      const float L = L_next, Dv = D_next;
      load_stats(item + gridDim.x);
      for (int j = 0; j < n_kv && ok; j++, g++) {
        const uint32_t buf = g & 1u;
        // phase A: probabilities of this thread's 64 columns from S alone
#ifdef FML_FA_PROFILE
        long long* const sprof = threadIdx.x == 64 ? p.prof : nullptr;
#else
        long long* const sprof = nullptr;
        (void)sprof;
#endif
        FA_STAMP(sprof, g, 0);
        ok = mbar_wait_warp(bar(C_SFULL + buf), (g >> 1) & 1u, abort_flag, p.status, 33);
        if (!ok) break;
        FA_STAMP(sprof, g, 1);
        tc_fence_after();
        const int lim = (p.causal && j == qb) ? row + 1 : BKV;
#pragma unroll
        for (int ci = 0; ci < 2; ci++) {
          const int c = half + 2 * ci;
          tmem_ld32(lane_addr + TM_S + buf * 128 + c * 32, tv);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; e++)
            pr[ci * 32 + e] = (c * 32 + e < lim) ? fa_exp2(fmaf(__uint_as_float(tv[e]), p.k2, -L)) * p.scale : 0.f;
        }
        tc_fence_before();
        mbar_arrive_warp(bar(C_SEMPTY + buf));
        FA_STAMP(sprof, g, 2);
        FA_STAMP(sprof, g, 3);
        // phase B: dS over dP
        ok = mbar_wait_warp(bar(C_DPFULL), g & 1u, abort_flag, p.status, 34);
        if (!ok) break;
        FA_STAMP(sprof, g, 4);
        tc_fence_after();
#pragma unroll
        for (int ci = 0; ci < 2; ci++) {
          const int c = half + 2 * ci;
          tmem_ld32(lane_addr + TM_DP + c * 32, tv);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; e++) tv[e] = __float_as_uint(fa_round_tf32(pr[ci * 32 + e] * (__uint_as_float(tv[e]) - Dv)));
          tmem_st32(lane_addr + TM_DP + c * 32, tv);
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive_warp(bar(C_DSFULL));
        FA_STAMP(sprof, g, 5);
        if (pending) {   // the finished item's tile, now that this item's first dS is published (off the operand's path)
          ok = flush_dq();
          if (!ok) break;
        }
      }
      if (ok) pending = true;
    }
    if (ok && pending) ok = flush_dq();
  }
  FA_TOTAL_END(p.prof);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------------------
// Backward, second kernel: dK and dV of one block of 128 keys, accumulated over the 128-query blocks that see it.
// The contraction of both products runs over the queries, so the tensor core needs P^T and dS^T with the KEY
// index on the TMEM lanes.  The kernel therefore rebuilds the scores transposed, S^T = K_j.Q_i^T and
// dP^T = V_j.dO_i^T (both operands K-major); each thread (= one key) turns its row of S^T into P^T and its row of
// dP^T into dS^T IN PLACE in tensor memory, from the saved row statistics of the queries, and the accumulating products
//   dV_j += P^T . dO_i      dK_j += dS^T . Q_i        (dO_i and Q_i as MN-major B operands)
// read their A operand from there.  Nothing score-sized touches shared or global memory.
// Order on the tensor pipe: ... dP^T_i, S^T_{i+1}, dV_i, dK_i, dP^T_{i+1} ...: the next block's scores are issued before
// the issuer waits for this block's P^T, so its exponentials run under dV_i and dK_i; dP^T_{i+1} overwrites dS^T_i after
// dK_i has read it, and S^T_{i+2} overwrites P^T_i after dV_i (issue order, no barrier).
// Shared memory (224 KiB): K_j, V_j (resident), Q_i, dO_i as K-major and as MN-major tiles, 32 KiB each; the producer
// refills each of the four per-block tiles in the order in which the pipe releases them (Q_i runs one block ahead);
// 32 KiB staging tile through which the store warp writes dV, then dK, of a finished item with tile stores.
// TMEM: S^T/P^T [0,128) and [128,256), dP^T/dS^T [256,384), dV [384,448), dK [448,512).
constexpr uint32_t CO_K = 0, CO_V = 32768, CO_Q = 65536, CO_DO = 98304, CO_QMN = 131072, CO_DOMN = 163840, CO_ST = 196608, CO_BAR = 229376;
constexpr int FA2_SMEM = CO_BAR + 256 + 1024;
constexpr uint32_t T2_ST = 0, T2_DPT = 256, T2_DV = 384, T2_DK = 448;
enum { D_KFULL = 0, D_KEMPTY, D_VFULL, D_VEMPTY, D_QKFULL, D_QKEMPTY, D_DOKFULL, D_DOKEMPTY, D_QMNFULL, D_QMNEMPTY, D_DOMNFULL,
       D_DOMNEMPTY, D_STFULL /* two */, D_STFULL1, D_DPTFULL, D_PTFULL, D_DSTFULL, D_DVDONE, D_ACCDONE, D_STAGED, D_STFREE, D_DVREAD, D_DKREAD, D_COUNT };

struct FaBwd2Params {
  int S, H, n_kb, causal;
  int n_items;
  float k2, scale;
  const float* lse;
  const float* dsum;
  float* dk; float* dv; long long ld;
  int accumulate;
  int* status;
  long long* prof;    // -DFML_FA_PROFILE builds, else NULL
};

__global__ void __launch_bounds__(FA_DKV_THREADS, 1)
attention_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                         const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                         const __grid_constant__ CUtensorMap tmQmn, const __grid_constant__ CUtensorMap tmDOmn,
                         const __grid_constant__ CUtensorMap tmDK, const __grid_constant__ CUtensorMap tmDV, const FaBwd2Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  auto bar = [&](int i) { return smem_base + CO_BAR + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + CO_BAR + 8 * D_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Persistent loop over (sequence, head, key block) items, heaviest first (key block 0 is seen by every query block).
  // u counts query blocks over all items of this CTA, it counts items; every barrier phase derives from them.
  const int n_bh = p.n_items / p.n_kb;
  const int n_q = p.S / BQ;
  auto item_coords = [&](int item, int& kbk, int& h, int& b, int& i0, int& n_it) {
    // CTAs walk the item list in alternating directions from round to round (full rounds only), which evens out the block
    // counts: with plain striding CTA c gets the same rank in every round and the heaviest CTAs end 4 % above the mean.
    {
      const int G = gridDim.x, k = item / G;
      if ((k & 1) && k < p.n_items / G) item = k * G + (G - 1 - (item - k * G));
    }
    kbk = item / n_bh;
    const int bh = item - kbk * n_bh;
    h = bh % p.H;
    b = bh / p.H;
    i0 = p.causal ? kbk : 0;   // first query block that sees this key block
    n_it = n_q - i0;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < D_COUNT; i++)
      mbar_init(bar(i), (i == D_PTFULL || i == D_DSTFULL || i == D_STAGED || i == D_DVREAD || i == D_DKREAD) ? 16u : 1u);   // warps (mbar_arrive_warp)
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  FA_TOTAL_BEGIN();

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      // cursor of the K-major Q tile (and, at the first block of an item, of K_j): one block ahead of the other loads
      int q_item = blockIdx.x, q_i = 0, q_nit = 0, q_kbk = 0, q_h = 0, q_b = 0, q_i0 = 0;
      uint32_t q_u = 0, q_it = 0;
      if (q_item < p.n_items) item_coords(q_item, q_kbk, q_h, q_b, q_i0, q_nit);
      auto load_qk = [&]() {
        if (q_item >= p.n_items) return true;
        if (q_i == 0) {
          if (!mbar_wait(bar(D_KEMPTY), (q_it & 1u) ^ 1u, abort_flag, p.status, 41)) return false;   // previous item's last S^T
          mbar_expect_tx(bar(D_KFULL), BKV * DH * 4);
          for (int kb = 0; kb < 2; kb++) tma_load_4d(smem_base + CO_K + kb * 16384, &tmK, bar(D_KFULL), kb * 32, q_kbk * BKV, q_h, q_b);
        }
        if (!mbar_wait(bar(D_QKEMPTY), (q_u & 1u) ^ 1u, abort_flag, p.status, 31)) return false;
        mbar_expect_tx(bar(D_QKFULL), BQ * DH * 4);
        for (int kb = 0; kb < 2; kb++) tma_load_4d(smem_base + CO_Q + kb * 16384, &tmQ, bar(D_QKFULL), kb * 32, (q_i0 + q_i) * BQ, q_h, q_b);
        q_u++;
        if (++q_i == q_nit) {
          q_item += gridDim.x;
          q_it++;
          q_i = 0;
          if (q_item < p.n_items) item_coords(q_item, q_kbk, q_h, q_b, q_i0, q_nit);
        }
        return true;
      };
      ok = load_qk();
      uint32_t u = 0, it = 0;
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, it++) {
        int kbk, h, b, i0, n_it;
        item_coords(item, kbk, h, b, i0, n_it);
        for (int i = 0; i < n_it && ok; i++, u++) {
          const uint32_t ph = u & 1u;
          const int q0 = (i0 + i) * BQ;
          if (i == 0) {
            ok = mbar_wait(bar(D_VEMPTY), (it & 1u) ^ 1u, abort_flag, p.status, 42);   // previous item's last dP^T
            if (!ok) break;
            mbar_expect_tx(bar(D_VFULL), BKV * DH * 4);
            for (int kb = 0; kb < 2; kb++) tma_load_4d(smem_base + CO_V + kb * 16384, &tmV, bar(D_VFULL), kb * 32, kbk * BKV, h, b);
          }
          ok = mbar_wait(bar(D_DOKEMPTY), ph ^ 1u, abort_flag, p.status, 43);
          if (!ok) break;
          mbar_expect_tx(bar(D_DOKFULL), BQ * DH * 4);
          for (int kb = 0; kb < 2; kb++) tma_load_4d(smem_base + CO_DO + kb * 16384, &tmDO, bar(D_DOKFULL), kb * 32, q0, h, b);
          ok = load_qk();   // Q of the NEXT block: its tile is released by S^T of this block, before dV / dK of the previous one
          if (!ok) break;
          ok = mbar_wait(bar(D_DOMNEMPTY), ph ^ 1u, abort_flag, p.status, 44);
          if (!ok) break;
          mbar_expect_tx(bar(D_DOMNFULL), BQ * DH * 4);
          for (int c = 0; c < 4; c++) tma_load_5d(smem_base + CO_DOMN + c * 8192, &tmDOmn, bar(D_DOMNFULL), 0, q0 + 32 * c, 0, h, b);
          ok = mbar_wait(bar(D_QMNEMPTY), ph ^ 1u, abort_flag, p.status, 39);
          if (!ok) break;
          mbar_expect_tx(bar(D_QMNFULL), BQ * DH * 4);
          for (int c = 0; c < 4; c++) tma_load_5d(smem_base + CO_QMN + c * 8192, &tmQmn, bar(D_QMNFULL), 0, q0 + 32 * c, 0, h, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_st = fa_idesc(BKV, BQ, 0, 0), idesc_acc = fa_idesc(BKV, DH, 0, 1);
      bool ok = true;
      // cursor of the next S^T product: one block ahead of the other three products, across items
      int s_item = blockIdx.x, s_i = 0, s_nit = 0;
      uint32_t s_u = 0, s_it = 0;
      if (s_item < p.n_items) { int a, b2, c, d2; item_coords(s_item, a, b2, c, d2, s_nit); }
      auto issue_st = [&]() {
        if (s_item >= p.n_items) return true;
        const uint32_t bf = s_u & 1u;
        if (s_i == 0 && !mbar_wait(bar(D_KFULL), s_it & 1u, abort_flag, p.status, 32)) return false;
        if (!mbar_wait(bar(D_QKFULL), s_u & 1u, abort_flag, p.status, 33)) return false;
        tc_fence_after();
        for (int kb = 0; kb < 2; kb++) {
          const uint64_t ak = make_smem_desc(smem_base + CO_K + kb * 16384, 16u, 1024u, 2u);
          const uint64_t bq = make_smem_desc(smem_base + CO_Q + kb * 16384, 16u, 1024u, 2u);
#pragma unroll
          for (int k = 0; k < 4; k++) umma_tf32(tmem_base + T2_ST + bf * 128, ak + 2u * k, bq + 2u * k, idesc_st, (kb | k) ? 1u : 0u);
        }
        umma_commit(bar(D_STFULL + bf));
        umma_commit(bar(D_QKEMPTY));
        s_u++;
        if (++s_i == s_nit) {          // last S^T of the item: K_j may be replaced
          umma_commit(bar(D_KEMPTY));
          s_item += gridDim.x;
          s_it++;
          s_i = 0;
          if (s_item < p.n_items) { int a, b2, c, d2; item_coords(s_item, a, b2, c, d2, s_nit); }
        }
        return true;
      };
      uint32_t u = 0, it = 0;
      ok = issue_st();
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, it++) {
        int kbk, h, b, i0, n_it;
        item_coords(item, kbk, h, b, i0, n_it);
        for (int i = 0; i < n_it && ok; i++, u++) {
          const uint32_t ph = u & 1u, bf = u & 1u;
          FA_STAMP(p.prof, u, 8);
          if (i == 0) ok = mbar_wait(bar(D_VFULL), it & 1u, abort_flag, p.status, 34);
          ok = ok && mbar_wait(bar(D_DOKFULL), ph, abort_flag, p.status, 45);
          if (!ok) break;
          FA_STAMP(p.prof, u, 9);
          tc_fence_after();
          for (int kb = 0; kb < 2; kb++) {
            const uint64_t av = make_smem_desc(smem_base + CO_V + kb * 16384, 16u, 1024u, 2u);
            const uint64_t bd = make_smem_desc(smem_base + CO_DO + kb * 16384, 16u, 1024u, 2u);
#pragma unroll
            for (int k = 0; k < 4; k++) umma_tf32(tmem_base + T2_DPT, av + 2u * k, bd + 2u * k, idesc_st, (kb | k) ? 1u : 0u);
          }
          umma_commit(bar(D_DPTFULL));
          umma_commit(bar(D_DOKEMPTY));
          if (i == n_it - 1) umma_commit(bar(D_VEMPTY));
          FA_STAMP(p.prof, u, 10);
          if (s_u == u + 1) ok = issue_st();   // S^T of the next block: its exponentials overlap dV and dK of this one
          if (!ok) break;
          FA_STAMP(p.prof, u, 11);
          ok = mbar_wait(bar(D_PTFULL), ph, abort_flag, p.status, 35) && mbar_wait(bar(D_DOMNFULL), ph, abort_flag, p.status, 40);
          // the first dV product of an item overwrites the accumulator: the compute warps must have read the previous item's
          if (ok && i == 0 && it > 0) ok = mbar_wait(bar(D_DVREAD), (it - 1) & 1u, abort_flag, p.status, 52);
          if (!ok) break;
          FA_STAMP(p.prof, u, 12);
          tc_fence_after();
          for (int c = 0; c < 4; c++) {   // 32 queries per chunk, 8 per instruction; A operand = P^T in tensor memory
            const uint64_t bdo = make_smem_desc(smem_base + CO_DOMN + c * 8192, 4096u, 512u, 1u);
#pragma unroll
            for (int k = 0; k < 4; k++)
              umma_tf32_ts(tmem_base + T2_DV, tmem_base + T2_ST + bf * 128 + c * 32 + k * 8, bdo + 64u * k, idesc_acc, (i | c | k) ? 1u : 0u);
          }
          umma_commit(bar(D_DOMNEMPTY));
          umma_commit(bar(D_DVDONE));
          FA_STAMP(p.prof, u, 13);
          ok = mbar_wait(bar(D_DSTFULL), ph, abort_flag, p.status, 46) && mbar_wait(bar(D_QMNFULL), ph, abort_flag, p.status, 47);
          if (ok && i == 0 && it > 0) ok = mbar_wait(bar(D_DKREAD), (it - 1) & 1u, abort_flag, p.status, 53);   // likewise for dK
          if (!ok) break;
          FA_STAMP(p.prof, u, 14);
          tc_fence_after();
          for (int c = 0; c < 4; c++) {
            const uint64_t bq = make_smem_desc(smem_base + CO_QMN + c * 8192, 4096u, 512u, 1u);
#pragma unroll
            for (int k = 0; k < 4; k++)
              umma_tf32_ts(tmem_base + T2_DK, tmem_base + T2_DPT + c * 32 + k * 8, bq + 64u * k, idesc_acc, (i | c | k) ? 1u : 0u);
          }
          umma_commit(bar(D_ACCDONE));
          umma_commit(bar(D_QMNEMPTY));
          FA_STAMP(p.prof, u, 15);
        }
      }
    }
  } else if (warp == FA_DKV_THREADS / 32 - 1) {
    // ------------------------------------------------------------------ store warp: dV, then dK, of every finished item
    if (lane == 0) {
      bool ok = true;
      uint32_t n = 0;
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x) {
        int kbk, h, b, i0, n_it;
        item_coords(item, kbk, h, b, i0, n_it);
        for (int which = 0; which < 2 && ok; which++, n++) {
          ok = mbar_wait(bar(D_STAGED), n & 1u, abort_flag, p.status, 48);   // the whole tile is in shared memory
          if (!ok) break;
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          const CUtensorMap* tm = which ? &tmDK : &tmDV;
          for (int kb = 0; kb < 2; kb++) {
            if (p.accumulate) tma_reduce_add_4d(tm, smem_base + CO_ST + kb * 16384, kb * 32, kbk * BKV, h, b);
            else tma_store_4d(tm, smem_base + CO_ST + kb * 16384, kb * 32, kbk * BKV, h, b);
          }
          tma_store_commit();
          tma_store_wait_read();          // the staging tile has been read and may be overwritten
          mbar_arrive(bar(D_STFREE));
        }
      }
    }
  } else {
    const int q4 = warp & 3;
    const int part = (warp - 2) >> 2;          // which 32-query chunk of every block, and which 16 columns of dV / dK
    const int row = q4 * 32 + lane;            // key inside the block
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q4 * 32) << 16);
    bool ok = true;
    uint32_t tv[32];
    float prs[32];
    uint32_t u = 0, n_st = 0;
    bool pending = false;        // a finished item whose dV / dK tiles are still to be read
    // The tiles of a finished item are read AFTER this thread has published the next item's first P^T / dS^T (the issuer
    // holds the first overwriting product back until all warps have read: D_DVREAD, D_DKREAD), so that reading, staging
    // and storing them is off the path from an operand to its product; measured with the reads in front of the
    // publication, an item boundary cost 5000 cycles, as much as a whole block.  Sixteen compute warps: with eight, the
    // same ordering gained nothing (293 us for the backward pass); with sixteen the boundary shrinks to about 1400 cycles
    // although the products of the steady state get slower (126 against 104 cycles per instruction), 278 us in all.
    auto flush_tile = [&](int which) {
      if (!mbar_wait_warp(bar(which ? D_ACCDONE : D_DVDONE), (u - 1) & 1u, abort_flag, p.status, which ? 38 : 51)) return false;
      tc_fence_after();
      uint32_t t16[16];
      tmem_ld16(lane_addr + (which ? T2_DK : T2_DV) + part * 16, t16);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive_warp(bar(which ? D_DKREAD : D_DVREAD));
      if (!mbar_wait_warp(bar(D_STFREE), (n_st & 1u) ^ 1u, abort_flag, p.status, 49)) return false;   // previous tile stored
      uint8_t* srow = smem_gen + CO_ST + (part >> 1) * 16384 + row * 128;   // K-major tile layout: 128-byte rows, chunks swizzled
#pragma unroll
      for (int i = 0; i < 4; i++)
        *reinterpret_cast<float4*>(srow + ((((part & 1) * 4 + i) ^ (row & 7)) << 4)) =
            make_float4(__uint_as_float(t16[4 * i]), __uint_as_float(t16[4 * i + 1]), __uint_as_float(t16[4 * i + 2]), __uint_as_float(t16[4 * i + 3]));
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive_warp(bar(D_STAGED));
      n_st++;
      return true;
    };
    for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x) {
      int kbk, h, b, i0, n_it;
      item_coords(item, kbk, h, b, i0, n_it);
      const int kj = kbk * BKV + row;            // key position in the sequence
      const long long stat_base = ((long long)b * p.H + h) * p.S;
      for (int i = 0; i < n_it && ok; i++, u++) {
        const uint32_t bf = u & 1u;
        const int q0 = (i0 + i) * BQ;
        if (lane < 8 && part == 0 && i + 1 < n_it) {   // statistics of the next query block (2 x 512 bytes): the loads below then hit the cache
          const float* nx = (lane < 4 ? p.lse : p.dsum) + stat_base + q0 + BQ + (lane & 3) * 32;
          asm volatile("prefetch.global.L2 [%0];" ::"l"(nx));
        }
        // phase A: P^T over S^T.  The row statistics of the queries are the same addresses for every lane (one
        // transaction per warp, L1 hits).
#ifdef FML_FA_PROFILE
        long long* const sprof = threadIdx.x == 64 ? p.prof : nullptr;
#else
        long long* const sprof = nullptr;
        (void)sprof;
#endif
        FA_STAMP(sprof, u, 0);
        ok = mbar_wait_warp(bar(D_STFULL + bf), (u >> 1) & 1u, abort_flag, p.status, 36);
        if (!ok) break;
        FA_STAMP(sprof, u, 1);
        tc_fence_after();
        {
          const uint32_t ta = lane_addr + T2_ST + bf * 128 + part * 32;
          tmem_ld32(ta, tv);
          tmem_ld_wait();
          const float4* Lp = reinterpret_cast<const float4*>(p.lse + stat_base + q0 + part * 32);
#pragma unroll
          for (int ch = 0; ch < 8; ch++) {
            const float4 L4 = __ldg(Lp + ch);
            const float* Le = reinterpret_cast<const float*>(&L4);
#pragma unroll
            for (int e = 0; e < 4; e++) {
              const int col = part * 32 + ch * 4 + e;            // query inside the block
              const bool vis = !p.causal || (q0 + col >= kj);
              const float pr = vis ? fa_exp2(fmaf(__uint_as_float(tv[ch * 4 + e]), p.k2, -Le[e])) : 0.f;
              prs[ch * 4 + e] = pr * p.scale;
              tv[ch * 4 + e] = __float_as_uint(fa_round_tf32(pr));
            }
          }
          tmem_st32(ta, tv);
        }
        tmem_st_wait();
        tc_fence_before();
        FA_STAMP(sprof, u, 2);
        mbar_arrive_warp(bar(D_PTFULL));
        FA_STAMP(sprof, u, 3);
        if (pending) {
          ok = flush_tile(0);
          if (!ok) break;
        }
        // phase B: dS^T over dP^T
        ok = mbar_wait_warp(bar(D_DPTFULL), u & 1u, abort_flag, p.status, 37);
        if (!ok) break;
        FA_STAMP(sprof, u, 4);
        tc_fence_after();
        {
          const uint32_t ta = lane_addr + T2_DPT + part * 32;
          tmem_ld32(ta, tv);
          tmem_ld_wait();
          const float4* Dp = reinterpret_cast<const float4*>(p.dsum + stat_base + q0 + part * 32);
#pragma unroll
          for (int ch = 0; ch < 8; ch++) {
            const float4 D4 = __ldg(Dp + ch);
            const float* De = reinterpret_cast<const float*>(&D4);
#pragma unroll
            for (int e = 0; e < 4; e++)
              tv[ch * 4 + e] = __float_as_uint(fa_round_tf32(prs[ch * 4 + e] * (__uint_as_float(tv[ch * 4 + e]) - De[e])));
          }
          tmem_st32(ta, tv);
        }
        tmem_st_wait();
        tc_fence_before();
        FA_STAMP(sprof, u, 5);
        mbar_arrive_warp(bar(D_DSTFULL));
        FA_STAMP(sprof, u, 6);
        if (pending) {
          ok = flush_tile(1);
          if (!ok) break;
          pending = false;
        }
      }
      if (ok && n_it > 0) pending = true;
    }
    if (ok && pending) ok = flush_tile(0) && flush_tile(1);
  }
  FA_TOTAL_END(p.prof);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// D[b][h][i] = sum_c dO[b, i, h, c] * O[b, i, h, c]: 16 lanes per (row, head), float4 each
__global__ void attention_rowdot_kernel(const float* __restrict__ dout, long long ld_do, const float* __restrict__ out, long long ld_o,
                                        float* __restrict__ dsum, long long rows_total, int S, int H) {
  const long long item = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 4;   // (global row, head)
  const int part = threadIdx.x & 15;
  if (item >= rows_total * H) return;   // whole 16-lane groups leave together
  const long long r = item / H;
  const int h = (int)(item - r * H);
  const float4 a = *reinterpret_cast<const float4*>(dout + r * ld_do + h * DH + part * 4);
  const float4 o = *reinterpret_cast<const float4*>(out + r * ld_o + h * DH + part * 4);
  float v = a.x * o.x + a.y * o.y + a.z * o.z + a.w * o.w;
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off, 16);
  if (part == 0) {
    const long long bseq = r / S;
    dsum[(bseq * H + h) * S + (r - bseq * S)] = v;
  }
}

}  // namespace

extern "C" {

int32_t fml_attention_fwd(fml_ctx* ctx, const fml_attention_desc* d) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, d && d->q && d->k && d->v && d->out, "fml_attention_fwd: NULL buffer");
  FML_REQUIRE(ctx, d->n_seq > 0 && d->heads > 0 && d->seq_len > 0, "fml_attention_fwd: bad sizes");
  FML_REQUIRE(ctx, d->d_head == DH, "fml_attention_fwd: d_head must be 64");
  FML_REQUIRE(ctx, d->seq_len % BQ == 0, "fml_attention_fwd: seq_len must be a multiple of 128");
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  FML_REQUIRE(ctx, al16(d->q) && al16(d->k) && al16(d->v) && al16(d->out) && d->ld_qkv % 4 == 0 && d->ld_out % 4 == 0,
              "fml_attention_fwd: operands must be 16-byte aligned with row strides that are multiples of 4 floats");
  FML_REQUIRE(ctx, d->ld_qkv >= (int64_t)d->heads * DH && d->ld_out >= (int64_t)d->heads * DH, "fml_attention_fwd: row stride smaller than heads * 64");
  const int S = d->seq_len, H = d->heads, Bn = d->n_seq;
  CUtensorMap tmQ, tmK, tmV, tmO;
  int32_t rc;
  const int64_t s2 = (int64_t)S * d->ld_qkv;
  if ((rc = fml_tc_make_tmap(ctx, d->out, DH, S, d->ld_out, H, Bn, DH, (int64_t)S * d->ld_out, 32, BQ, false, 0, &tmO))) return rc;
  if ((rc = fml_tc_make_tmap(ctx, d->q, DH, S, d->ld_qkv, H, Bn, DH, s2, 32, BQ, false, 0, &tmQ))) return rc;
  if ((rc = fml_tc_make_tmap(ctx, d->k, DH, S, d->ld_qkv, H, Bn, DH, s2, 32, BKV, false, 0, &tmK))) return rc;
  if ((rc = fml_tc_make_tmap(ctx, d->v, DH, S, d->ld_qkv, H, Bn, DH, s2, 32, 32, true, 2, &tmV))) return rc;
  FaParams p;
  p.S = S; p.H = H; p.n_qb = S / BQ;
  p.causal = d->causal ? 1 : 0;
  p.k2 = d->scale * 1.4426950408889634f;
  p.out = d->out; p.ld_out = d->ld_out;
  p.lse = d->lse;
  p.status = ctx->d_status;
  FML_ONCE_PER_DEVICE(ctx, {
    FML_CUDA(ctx, cudaFuncSetAttribute(attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM));
    FML_CUDA(ctx, cudaFuncSetAttribute(attention_fwd_long_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM));
  });
  const long long items = (long long)Bn * H * p.n_qb;
  FML_REQUIRE(ctx, items <= 0x7fffffffLL, "fml_attention_fwd: too many work items");
  p.n_items = (int)items;
  p.round_p = getenv("FML_FA_NOROUND") ? 0 : 1;
  const unsigned grid = (unsigned)std::min<long long>(items, ctx->sm_count);
  p.prof = nullptr;
#ifdef FML_FA_PROFILE
  static long long* prof_buf = nullptr;
  static int prof_calls = 0;
  if (!prof_buf) { cudaMalloc(&prof_buf, 512 * sizeof(long long)); }
  cudaMemsetAsync(prof_buf, 0, 512 * sizeof(long long), ctx->stream);
  p.prof = prof_buf;
#endif
  if (S <= FA_MAX_SEQ_TMEM_P) attention_fwd_kernel<<<grid, FA_THREADS, FA_SMEM, ctx->stream>>>(tmQ, tmK, tmV, tmO, p);
  else attention_fwd_long_kernel<<<grid, FA_LONG_THREADS, FA_SMEM, ctx->stream>>>(tmQ, tmK, tmV, p);
  FML_LAUNCH_CHECK(ctx, "attention_fwd_kernel");
#ifdef FML_FA_PROFILE
  if (++prof_calls == 4) {
    long long h[512];
    cudaStreamSynchronize(ctx->stream);
    cudaMemcpy(h, prof_buf, sizeof h, cudaMemcpyDeviceToHost);
    fprintf(stderr, "attention fwd, CTA 0, key blocks 8..15, cycles relative to block 8's first stamp\n"
                    "softmax: top | S full | S loaded | max exchanged | max read | P formed | P published | item end;  issuer: top | next S issued | P,V ready | PV issued | last-of-item\n");
    const long long t0 = h[0];
    for (int g = 0; g < 8; g++) {
      fprintf(stderr, "g=%d sm:", g + 8);
      for (int k = 0; k < 8; k++) fprintf(stderr, " %lld", h[g * 16 + k] ? h[g * 16 + k] - t0 : -1);
      fprintf(stderr, "  is:");
      for (int k = 8; k < 12; k++) fprintf(stderr, " %lld", h[g * 16 + k] ? h[g * 16 + k] - t0 : -1);
      fprintf(stderr, " (next S operands ready %lld, O free %lld, P ready %lld) %s\n", h[g * 16 + 14] ? h[g * 16 + 14] - t0 : -1,
              h[g * 16 + 12] ? h[g * 16 + 12] - t0 : -1, h[g * 16 + 15] ? h[g * 16 + 15] - t0 : -1, h[g * 16 + 13] ? "last" : "");
    }
    fprintf(stderr, "per softmax warp (2..17): arrival at block 12 | P_12 published | P_13 published\n");
    for (int w = 2; w < 18; w++) fprintf(stderr, "  w%d: %lld %lld %lld\n", w, h[464 + w] - t0, h[424 + w] - t0, h[444 + w] - t0);
    {
      long long cmin = 1LL << 62, cmax = 0, csum = 0, nmax = 0;
      int n = 0;
      for (int c = 0; c < 148; c++) {
        const long long cy = h[128 + 2 * c], ns = h[129 + 2 * c];
        if (!cy) continue;
        n++; csum += cy; cmin = cy < cmin ? cy : cmin; cmax = cy > cmax ? cy : cmax; nmax = ns > nmax ? ns : nmax;
      }
      if (n) fprintf(stderr, "per-CTA cycles over %d CTAs: min %lld avg %lld max %lld; longest CTA %lld ns; CTA 0: %lld cycles in %lld ns = %.3f GHz\n",
                     n, cmin, csum / n, cmax, nmax, h[128], h[129], (double)h[128] / (double)h[129]);
    }
  }
#endif
  return FML_OK;
}


int32_t fml_attention_bwd(fml_ctx* ctx, const fml_attention_desc* d, const float* dout, int64_t ld_dout, float* dq, float* dk,
                          float* dv, int64_t ld_dqkv, int32_t accumulate, float* scratch) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, d && d->q && d->k && d->v && d->out && d->lse && dout && dq && dk && dv && scratch, "fml_attention_bwd: NULL buffer");
  FML_REQUIRE(ctx, d->n_seq > 0 && d->heads > 0 && d->seq_len > 0 && d->d_head == DH && d->seq_len % BQ == 0,
              "fml_attention_bwd: d_head must be 64 and seq_len a multiple of 128");
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  FML_REQUIRE(ctx, al16(d->q) && al16(d->k) && al16(d->v) && al16(d->out) && al16(dout) && al16(dq) && al16(dk) && al16(dv) && al16(scratch) &&
                       d->ld_qkv % 4 == 0 && d->ld_out % 4 == 0 && ld_dout % 4 == 0 && ld_dqkv % 4 == 0,
              "fml_attention_bwd: operands must be 16-byte aligned with row strides that are multiples of 4 floats");
  const int S = d->seq_len, H = d->heads, Bn = d->n_seq;
  const long long rows = (long long)Bn * S;
  float* dsum = scratch;
  {
    const long long threads = rows * H * 16;
    attention_rowdot_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, ctx->stream>>>(dout, ld_dout, d->out, d->ld_out, dsum, rows, S, H);
    FML_LAUNCH_CHECK(ctx, "attention_rowdot_kernel");
  }
  CUtensorMap tmQ, tmDO, tmK, tmV, tmKmn, tmQmn, tmDOmn, tmDQ, tmDK, tmDV;
  int32_t rc;
  const int64_t s2 = (int64_t)S * d->ld_qkv, s2o = (int64_t)S * ld_dout;
  if ((rc = fml_tc_make_tmap(ctx, d->q, DH, S, d->ld_qkv, H, Bn, DH, s2, 32, BQ, false, 0, &tmQ))) return rc;
  if ((rc = fml_tc_make_tmap(ctx, dout, DH, S, ld_dout, H, Bn, DH, s2o, 32, BQ, false, 0, &tmDO))) return rc;
  if ((rc = fml_tc_make_tmap(ctx, d->k, DH, S, d->ld_qkv, H, Bn, DH, s2, 32, BKV, false, 0, &tmK))) return rc;
  if ((rc = fml_tc_make_tmap(ctx, d->v, DH, S, d->ld_qkv, H, Bn, DH, s2, 32, BKV, false, 0, &tmV))) return rc;
  if ((rc = fml_tc_make_tmap(ctx, d->k, DH, S, d->ld_qkv, H, Bn, DH, s2, 32, 32, true, 2, &tmKmn))) return rc;
  if ((rc = fml_tc_make_tmap(ctx, d->q, DH, S, d->ld_qkv, H, Bn, DH, s2, 32, 32, true, 2, &tmQmn))) return rc;
  if ((rc = fml_tc_make_tmap(ctx, dq, DH, S, ld_dqkv, H, Bn, DH, (int64_t)S * ld_dqkv, 32, BQ, false, 0, &tmDQ))) return rc;
  if ((rc = fml_tc_make_tmap(ctx, dk, DH, S, ld_dqkv, H, Bn, DH, (int64_t)S * ld_dqkv, 32, BKV, false, 0, &tmDK))) return rc;
  if ((rc = fml_tc_make_tmap(ctx, dv, DH, S, ld_dqkv, H, Bn, DH, (int64_t)S * ld_dqkv, 32, BKV, false, 0, &tmDV))) return rc;
  if ((rc = fml_tc_make_tmap(ctx, dout, DH, S, ld_dout, H, Bn, DH, s2o, 32, 32, true, 2, &tmDOmn))) return rc;
  FML_ONCE_PER_DEVICE(ctx, {
    FML_CUDA(ctx, cudaFuncSetAttribute(attention_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM));
    FML_CUDA(ctx, cudaFuncSetAttribute(attention_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA2_SMEM));
  });
  const unsigned grid = (unsigned)((long long)Bn * H * (S / BQ));
  FaBwdParams p;
  p.S = S; p.H = H; p.n_qb = S / BQ; p.causal = d->causal ? 1 : 0;
  p.scale = d->scale; p.k2 = d->scale * 1.4426950408889634f;
  p.lse = d->lse; p.dsum = dsum;
  p.dq = dq; p.ld_dq = ld_dqkv; p.accumulate = accumulate ? 1 : 0;
  p.status = ctx->d_status;
  p.n_items = (int)grid;
  p.prof = nullptr;
#ifdef FML_FA_PROFILE
  static long long* prof_buf = nullptr;
  static int prof_calls = 0;
  if (!prof_buf) { cudaMalloc(&prof_buf, 512 * sizeof(long long)); }
  cudaMemsetAsync(prof_buf, 0, 512 * sizeof(long long), ctx->stream);
  p.prof = prof_buf;
#endif
  attention_bwd_dq_kernel<<<std::min<unsigned>(grid, (unsigned)ctx->sm_count), FA_BWD_THREADS, FA_SMEM, ctx->stream>>>(tmQ, tmDO, tmK, tmV, tmKmn, tmDQ, p);
  FML_LAUNCH_CHECK(ctx, "attention_bwd_dq_kernel");
#ifdef FML_FA_PROFILE
  ++prof_calls;
  if (prof_calls == 4) {
    long long h[512];
    cudaStreamSynchronize(ctx->stream);
    cudaMemcpy(h, prof_buf, sizeof h, cudaMemcpyDeviceToHost);
    fprintf(stderr, "attention bwd dQ, CTA 0, key blocks 8..15, cycles relative to block 8's first stamp\n"
                    "compute: top | S full | P formed | dQ flushed | dP full | dS published;  issuer: top | V,dO ready | dP issued | next K ready | next S issued | dS,K ready | dQ issued | last-of-item\n");
    const long long t0 = h[0];
    for (int g = 0; g < 8; g++) {
      fprintf(stderr, "g=%d cp:", g + 8);
      for (int k = 0; k < 6; k++) fprintf(stderr, " %lld", h[g * 16 + k] ? h[g * 16 + k] - t0 : -1);
      fprintf(stderr, "  is:");
      for (int k = 8; k < 15; k++) fprintf(stderr, " %lld", h[g * 16 + k] ? h[g * 16 + k] - t0 : -1);
      fprintf(stderr, " %s\n", h[g * 16 + 15] ? "last" : "");
    }
    {
      long long cmin = 1LL << 62, cmax = 0, csum = 0, nmax = 0;
      int n = 0;
      for (int c = 0; c < 148; c++) {
        const long long cy = h[128 + 2 * c], ns = h[129 + 2 * c];
        if (!cy) continue;
        n++; csum += cy; cmin = cy < cmin ? cy : cmin; cmax = cy > cmax ? cy : cmax; nmax = ns > nmax ? ns : nmax;
      }
      if (n) fprintf(stderr, "per-CTA cycles over %d CTAs: min %lld avg %lld max %lld; longest CTA %lld ns; CTA 0: %lld cycles in %lld ns = %.3f GHz\n",
                     n, cmin, csum / n, cmax, nmax, h[128], h[129], (double)h[128] / (double)h[129]);
    }
  }
#endif
  FaBwd2Params p2;
  p2.S = S; p2.H = H; p2.n_kb = S / BKV; p2.causal = p.causal;
  p2.k2 = p.k2; p2.scale = p.scale; p2.lse = d->lse; p2.dsum = dsum;
  p2.dk = dk; p2.dv = dv; p2.ld = ld_dqkv; p2.accumulate = p.accumulate;
  p2.status = ctx->d_status;
  p2.n_items = (int)grid;
  p2.prof = nullptr;
#ifdef FML_FA_PROFILE
  static long long* prof_buf2 = nullptr;
  if (!prof_buf2) { cudaMalloc(&prof_buf2, 512 * sizeof(long long)); }
  cudaMemsetAsync(prof_buf2, 0, 512 * sizeof(long long), ctx->stream);
  p2.prof = prof_buf2;
#endif
  attention_bwd_dkv_kernel<<<std::min<unsigned>(grid, (unsigned)ctx->sm_count), FA_DKV_THREADS, FA2_SMEM, ctx->stream>>>(tmK, tmV, tmQ, tmDO, tmQmn,
                                                                                                                    tmDOmn, tmDK, tmDV, p2);
  FML_LAUNCH_CHECK(ctx, "attention_bwd_dkv_kernel");
#ifdef FML_FA_PROFILE
  if (prof_calls == 4) {
    long long h[512];
    cudaStreamSynchronize(ctx->stream);
    cudaMemcpy(h, prof_buf2, sizeof h, cudaMemcpyDeviceToHost);
    fprintf(stderr, "attention bwd dK/dV, CTA 0, query blocks 8..15, cycles relative to block 8's first stamp\n"
                    "compute: top | S^T full | P^T stored | P^T published | dP^T full | dS^T stored | dS^T published;  issuer: top | V,dO ready | dP^T issued | next S^T issued | P^T,dO ready | dV issued | dS^T,Q ready | dK issued\n");
    const long long t0 = h[0];
    for (int g = 0; g < 8; g++) {
      fprintf(stderr, "u=%d cp:", g + 8);
      for (int k = 0; k < 7; k++) fprintf(stderr, " %lld", h[g * 16 + k] ? h[g * 16 + k] - t0 : -1);
      fprintf(stderr, "  is:");
      for (int k = 8; k < 16; k++) fprintf(stderr, " %lld", h[g * 16 + k] ? h[g * 16 + k] - t0 : -1);
      fprintf(stderr, "\n");
    }
    long long cmin = 1LL << 62, cmax = 0, csum = 0;
    int n = 0;
    for (int c = 0; c < 148; c++) {
      const long long cy = h[128 + 2 * c];
      if (!cy) continue;
      n++; csum += cy; cmin = cy < cmin ? cy : cmin; cmax = cy > cmax ? cy : cmax;
    }
    if (n) fprintf(stderr, "per-CTA cycles over %d CTAs: min %lld avg %lld max %lld; CTA 0: %lld cycles in %lld ns\n", n, cmin, csum / n, cmax, h[128], h[129]);
  }
#endif
  return FML_OK;
}

}  // extern "C"
