// Dense contraction on the Blackwell tensor cores: tcgen05.mma kind::tf32 with the
// accumulator in TMEM, operands staged in shared memory by TMA, a warp-specialised
// producer / MMA-issuer / epilogue pipeline and a persistent tile loop.
//
// One CTA = 320 threads:
//   warp 0      TMA producer   (one lane issues cp.async.bulk.tensor per stage)
//   warp 1      MMA issuer     (one lane issues tcgen05.mma; the warp owns TMEM alloc/free)
//   warps 2..9  epilogue       (tcgen05.ld -> bias/activation -> global stores); warp w reads the TMEM
//                              lane quarter w % 4, and the two warps of a quarter take alternate
//                              32-column blocks (the epilogue is instruction-latency bound: these are
//                              the only busy warps of their schedulers)
// Tile: 128 (M) x BN (N, 64/128/256) x 32 (K, one 128-byte swizzle row of fp32).
// TMEM holds two accumulators (columns [0,256) and [256,512)) so the epilogue of tile i
// overlaps the main loop of tile i+1.
//
// Operand layouts.  op(A)[M x K] and op(B)[K x N] can each be stored K-contiguous
// ("K-major": A not transposed, B transposed) or M/N-contiguous ("MN-major").  Both are
// consumed in place, through the major-ness bits of the instruction descriptor:
//   K-major : one TMA box {32 k, rows} lands as rows x 128 B, 128B-swizzled;
//             descriptor SBO = 1024 B (8 rows), k-step of 8 elements = +32 B.
//   MN-major: boxes {32 m, 32 k} land as 32 k-rows x 128 B with the 32-byte-chunk swizzle
//             (CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B <-> UMMA SWIZZLE_128B_BASE32B, 4-row atoms);
//             block j of 32 m at +j*4096 B; descriptor LBO = 4096 B (next 32 m), SBO = 512 B
//             (next 4 k), k-step of 8 elements = +1024 B.
// So the reference's materialised transposes (tensor.dart:877-884, 908-915, 927-934) never exist.
//
// Two kernel shapes share the code (template parameter PAIR):
//   single  one CTA per 128 x BN tile, tcgen05 cta_group::1, 4 stages of 48 KiB.
//   pair    a cluster of two CTAs per 256 x 256 tile, tcgen05 cta_group::2: each CTA stages its own
//           128 rows of A and HALF of the B tile (128 columns), the leader CTA issues one
//           M = 256 MMA that reads both CTAs' shared memory, and each CTA keeps the accumulator
//           rows it owns in its own TMEM.  Shared-memory fill per flop drops by a third and the
//           ring grows to 6 stages of 32 KiB, which is what feeds the tensor pipe on large
//           problems.  Loads carry no multicast qualifier; the peer's loads signal the leader's
//           full barrier, and tcgen05.commit arrives on both CTAs' empty barriers.
//
// 3xTF32: a pre-pass writes hi = rna_tf32(x) and lo = x - hi for both operands into the
// context's scratch arena; the K loop then runs three segments (lo.hi, hi.lo, hi.hi) into the
// same accumulator, small terms first.
//
// Chunked accumulation.  The error of a long fp32 accumulation chain inside the tensor core grows
// linearly with K (measured in 3xTF32 mode: 8.7e-7 at K = 512, 6.8e-6 at 4096, 1.4e-5 at 8192).  When K
// exceeds the chunk length (1024 for 3xTF32, 8192 for TF32) the K loop is cut into chunks that
// alternate between the two TMEM accumulators; the epilogue warps drain each chunk and add it, in
// fp32 with round-to-nearest, into a per-CTA slab of the scratch arena (L2-resident), and the last
// chunk adds the slab back before the usual epilogue.  Draining overlaps the next chunk's MMAs.
//
// Split K.  A product with few output tiles and a long K (weight gradients: K = all tokens of the
// batch) would leave most SMs idle; its K range is then divided over several CTAs per tile, each of
// which adds its partial product into C with vector atomics (C is zeroed first unless beta = 1).  Only
// for plain products (no bias, activation or pre-activation output).  The order of the atomic adds
// is not fixed, so results can differ in the last fp32 bit between runs.
//
// Every wait on an mbarrier is bounded (2 s of %globaltimer); on expiry the kernel records a
// code in *status, raises a CTA-wide abort flag, and all roles fall through to the common
// tail, which frees TMEM.
#include <stdlib.h>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 32;
constexpr int A_STAGE_BYTES = BM * BK * 4;    // 16 KiB
template <bool PAIR> struct Cfg {
  // The operand ring holds RING_BYTES; a stage is 16 KiB of A plus 128 B per staged B column, so narrow
  // tiles get a deeper ring (BN = 256 single: 4 stages, pair or BN = 128: 7, BN = 64: 9), which is what
  // hides the load latency of short, latency-bound products.
  static constexpr int RING_BYTES = 7 * 32768;
  static constexpr int MAX_STAGES = 12;
  static constexpr int SMEM_BYTES = RING_BYTES + 1024 /*align*/ + 512 /*barriers*/;
};
constexpr int NUM_THREADS = 320;  // producer warp, issuer warp, 8 epilogue warps
constexpr uint32_t TMEM_COLS = 512;

struct TcParams {
  int M, N, K;
  int tiles_m, tiles_n, nb1, nb2;
  int BN;
  int a_mn, b_mn;  // 1 = MN-major operand
  int a_blk, b_blk;  // MN-major operand is loaded as ONE 5-D box of 32-column blocks (needs cols % 32 == 0)
  int nseg;        // 1 (TF32) or 3 (3xTF32)
  int nstages, stage_bytes;  // operand ring geometry
  int group_m;     // m-tiles per rasterisation group
  int kblocks;
  int kchunk;      // k-blocks accumulated in TMEM before the partial sum is drained (see 'chunked accumulation')
  int ksplit;      // > 1: the K range of a tile is divided over this many CTAs that add into C atomically
  int kb_per_split;
  float* partial;  // per-CTA slab [BN/32][128][32] for the drained partial sums (only when kblocks > kchunk)
  float* C;
  float* Z;
  const float* bias;
  long long ldc, sC1, sC2;
  int act;
  float alpha, beta;
  int* status;
  uint32_t idesc;
  const float* dact_saved;  // gradient epilogue: result *= act'(dact_saved) (same indexing as C)
  int dact;
  int rowop, rowop_causal;  // row epilogue over complete rows (attention): 1 softmax, 2 softmax backward
  const float* rowop_aux;
  int lstm;     // 1: LSTM gate epilogue (see fml_lstm_epilogue); C is not written
  fml_lstm_epilogue le;
  int debug;  // diagnostics builds only (-DFML_GEMM_DIAGNOSTICS): 1 = producer skips the TMA loads, 2 = issuer skips the MMAs
};

using namespace fml_tc;

// Tile index -> (batch, m-tile, n-tile); tiles are walked in groups of `group_m` m-tiles (all n-tiles of a
// group before the next group) so that the group's A panel stays in L2 while B streams past it.
__device__ __forceinline__ void tile_coords(const TcParams& p, int t, int& b, int& tm, int& tn) {
  const int per_batch = p.tiles_m * p.tiles_n;
  b = t / per_batch;
  int r = t - b * per_batch;
  if (p.rowop) {  // the n-tiles of a row block are consecutive: they fill the two accumulators of one CTA
    tm = r / p.tiles_n;
    tn = r - tm * p.tiles_n;
    return;
  }
  const int GROUP = p.group_m;
  int group_sz = GROUP * p.tiles_n;
  int g = r / group_sz;
  int first_m = g * GROUP;
  int gm = min(GROUP, p.tiles_m - first_m);
  int rr = r - g * group_sz;
  tm = first_m + rr % gm;
  tn = rr / gm;
}

template <bool PAIR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmAlo, const __grid_constant__ CUtensorMap tmBlo,
               const TcParams p) {
  constexpr int MAX_STAGES = Cfg<PAIR>::MAX_STAGES;
  constexpr int RING_BYTES = Cfg<PAIR>::RING_BYTES;
  const int STAGES = p.nstages;            // runtime: depends on the tile width
  const int STAGE_BYTES = p.stage_bytes;   // multiple of 1024
  constexpr int CTAS = PAIR ? 2 : 1;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128B swizzle pattern repeats every 8 rows x 128 B
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bars = smem_base + RING_BYTES;
  // barrier layout (8 bytes each): full[S], empty[S], tmem_full[2], tmem_empty[2], then tmem slot + abort flag
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (MAX_STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * MAX_STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * MAX_STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + RING_BYTES + 8 * (2 * MAX_STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // let the next kernel of the stream be scheduled as SMs free up (it parks at its own griddepcontrol.wait)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;  // 0 = leader of the pair
  const int unit = PAIR ? (blockIdx.x >> 1) : blockIdx.x;     // tile-loop start of this CTA (pair)
  const int unit_stride = PAIR ? (gridDim.x >> 1) : gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(full_bar(s), 1);   // the leader's arrive.expect_tx (+ transaction bytes of both CTAs)
      mbar_init(empty_bar(s), 1);  // one tcgen05.commit
    }
    for (int a = 0; a < 2; a++) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8 * CTAS);  // every epilogue warp of the pair
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Programmatic dependent launch: everything above (barrier init, TMEM allocation, the cluster handshake) touched
  // no global memory and may run while the previous kernel of the stream is still finishing; from here on this
  // kernel reads and writes tensors, so it first waits until that kernel has completed and its writes are visible.
  // A no-op when the launch did not ask for the overlap.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  const int num_tiles = p.tiles_m * p.tiles_n * p.nb1 * p.nb2;
  const int num_units = num_tiles * p.ksplit;  // work units: (tile, K split)
  // i-th work unit of this CTA (pair).  With a row epilogue a CTA takes the tiles_n consecutive tiles of a row block.
  auto nth_unit = [&](int i) {
    if (p.rowop) return (unit + (i / p.tiles_n) * unit_stride) * p.tiles_n + i % p.tiles_n;
    return unit + i * unit_stride;
  };
  // unit -> tile index, first k-block and number of k-blocks of its K range
  auto unit_range = [&](int u, int& tile, int& kb0, int& nkb) {
    const int split = u / num_tiles;
    tile = u - split * num_tiles;
    if (p.ksplit > 1) {
      // interleaved: split s owns k-blocks s, s + ksplit, ...  All splits then stream through the same
      // region of the operands at the same time (shared DRAM pages and L2 lines) instead of ksplit distant ones
      kb0 = 0;
      nkb = (p.kblocks - split + p.ksplit - 1) / p.ksplit;
    } else {
      kb0 = 0;
      nkb = p.kblocks;
    }
  };
  const int bn_cta = PAIR ? (p.BN >> 1) : p.BN;            // B columns this CTA stages
  const uint32_t b_stage_bytes = (uint32_t)bn_cta * BK * 4;
  const int tile_m = PAIR ? 2 * BM : BM;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int it_u = 0; ok; it_u++) {
        const int u = nth_unit(it_u);
        if (u >= num_units) break;
        int t, kb0, nkb, b, tm, tn;
        unit_range(u, t, kb0, nkb);
        tile_coords(p, t, b, tm, tn);
        const int b1 = b % p.nb1, b2 = b / p.nb1;
        const int m0 = tm * tile_m + (int)rank * BM;
        const int n0 = tn * p.BN + (int)rank * bn_cta;
        // iteration order: chunk, then segment, then k-block inside the chunk
        for (int kb_lo = kb0; kb_lo < kb0 + nkb && ok; kb_lo += p.kchunk) {
         const int kb_n = min(p.kchunk, kb0 + nkb - kb_lo);
         for (int seg = 0; seg < p.nseg && ok; seg++) {
         for (int kb = kb_lo; kb < kb_lo + kb_n; kb++) {
          ok = mbar_wait(empty_bar(s), ph ^ 1, abort_flag, p.status, 1);
          if (!ok) break;
          const int k0 = (p.ksplit > 1 ? (u / num_tiles) + kb * p.ksplit : kb) * BK;
          // 3xTF32 segments: (A_lo,B_hi), (A_hi,B_lo), (A_hi,B_hi); TF32: (A,B)
          const CUtensorMap* ta = (p.nseg == 3 && seg == 0) ? &tmAlo : &tmA;
          const CUtensorMap* tb = (p.nseg == 3 && seg == 1) ? &tmBlo : &tmB;
          const uint32_t sa = smem_base + s * STAGE_BYTES;
          const uint32_t sb = sa + A_STAGE_BYTES;
#ifdef FML_GEMM_DIAGNOSTICS
          if (p.debug & 1) {
            if (rank == 0) mbar_arrive(full_bar(s));
            if (++s == STAGES) { s = 0; ph ^= 1; }
            continue;
          }
#endif
          if (rank == 0) mbar_expect_tx(full_bar(s), CTAS * (A_STAGE_BYTES + b_stage_bytes));
          auto load = [&](uint32_t dst, const CUtensorMap* tmap, int c0, int c1) {
            if (PAIR) tma_load_4d_pair(dst, tmap, full_bar(s), c0, c1, b1, b2);
            else tma_load_4d(dst, tmap, full_bar(s), c0, c1, b1, b2);
          };
          // One TMA instruction costs ~64 issue cycles whatever its size, so an MN-major operand is
          // fetched as one 5-D box {32 columns, 32 k-rows, blocks} when its row length allows it.
          auto load_blocks = [&](uint32_t dst, const CUtensorMap* tmap, int c0) {
            if (PAIR) tma_load_5d_pair(dst, tmap, full_bar(s), 0, k0, c0 >> 5, b1, b2);
            else tma_load_5d(dst, tmap, full_bar(s), 0, k0, c0 >> 5, b1, b2);
          };
          if (p.a_mn) {
            if (p.a_blk) load_blocks(sa, ta, m0);
            else for (int j = 0; j < BM / 32; j++) load(sa + j * 4096, ta, m0 + 32 * j, k0);
          } else {
            load(sa, ta, k0, m0);
          }
          if (p.b_mn) {
            if (p.b_blk) load_blocks(sb, tb, n0);
            else for (int j = 0; j < bn_cta / 32; j++) load(sb + j * 4096, tb, n0 + 32 * j, k0);
          } else {
            load(sb, tb, k0, n0);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
         }
         }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      const uint32_t a_lbo = p.a_mn ? 4096u : 16u, b_lbo = p.b_mn ? 4096u : 16u;
      const uint32_t a_kstep = p.a_mn ? (1024u >> 4) : (32u >> 4);
      const uint32_t b_kstep = p.b_mn ? (1024u >> 4) : (32u >> 4);
      for (int it_u = 0; ok; it_u++) {
       const int u = nth_unit(it_u);
       if (u >= num_units) break;
       int t, kb0, nkb;
       unit_range(u, t, kb0, nkb);
       for (int kb_lo = kb0; kb_lo < kb0 + nkb && ok; kb_lo += p.kchunk) {
        ok = mbar_wait(tempty_bar(acc), acc_ph ^ 1, abort_flag, p.status, 2);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)acc * 256u;
        const int its = min(p.kchunk, kb0 + nkb - kb_lo) * p.nseg;
        for (int it = 0; it < its; it++) {
          ok = mbar_wait(full_bar(s), ph, abort_flag, p.status, 3);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_base + s * STAGE_BYTES;
          const uint32_t sb = sa + A_STAGE_BYTES;
          const uint64_t adesc = make_smem_desc(sa, a_lbo, p.a_mn ? 512u : 1024u, p.a_mn ? 1u : 2u);
          const uint64_t bdesc = make_smem_desc(sb, b_lbo, p.b_mn ? 512u : 1024u, p.b_mn ? 1u : 2u);
#ifdef FML_GEMM_DIAGNOSTICS
          if (p.debug & 2) {
            if (PAIR) mbar_arrive_remote(empty_bar(s), 1);
            mbar_arrive(empty_bar(s));
            if (++s == STAGES) { s = 0; ph ^= 1; }
            continue;
          }
#endif
#pragma unroll
          for (int k = 0; k < BK / 8; k++) {
            const uint64_t ad = adesc + (uint64_t)(k * a_kstep), bd = bdesc + (uint64_t)(k * b_kstep);
            const uint32_t accum = (it > 0 || k > 0) ? 1u : 0u;
            if (PAIR) umma_tf32_pair(tmem_d, ad, bd, p.idesc, accum);
            else umma_tf32(tmem_d, ad, bd, p.idesc, accum);
          }
          // frees the stage (in both CTAs of a pair) once these MMAs have read it
          if (PAIR) umma_commit_pair(empty_bar(s), 3);
          else umma_commit(empty_bar(s));
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        // accumulator (of this chunk) complete; each CTA of a pair holds its own 128 rows
        if (PAIR) umma_commit_pair(tfull_bar(acc), 3);
        else umma_commit(tfull_bar(acc));
        if (++acc == 2) { acc = 0; acc_ph ^= 1; }
       }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;            // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;  // two warps share a quarter and take alternate 32-column blocks
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    const bool vec_ok = ((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                        ((p.sC1 & 3) == 0) && ((p.sC2 & 3) == 0) &&
                        (p.Z == nullptr || (reinterpret_cast<uintptr_t>(p.Z) & 15) == 0) &&
                        (p.bias == nullptr || (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0) &&
                        (p.dact_saved == nullptr || (reinterpret_cast<uintptr_t>(p.dact_saved) & 15) == 0);
    const bool plain = !p.bias && p.alpha == 1.f && p.act == FML_ACT_NONE && !p.Z && p.beta == 0.f && p.ksplit == 1 && !p.dact_saved;
    for (int it_u = 0; ok; it_u++) {
      const int u = nth_unit(it_u);
      if (u >= num_units) break;
      int t, kb0, nkb, b, tm, tn;
      unit_range(u, t, kb0, nkb);
      tile_coords(p, t, b, tm, tn);
      const int b1 = b % p.nb1, b2 = b / p.nb1;
      const int m0 = tm * tile_m + (int)rank * BM, n0 = tn * p.BN;
      if (p.rowop) {
        // ---- row epilogue: the complete rows of this 128-row block sit in TMEM (one or both accumulators)
        int accs[2];
        for (int j = 0; j < p.tiles_n && ok; j++) {
          accs[j] = acc;
          ok = mbar_wait(tfull_bar(acc), acc_ph, abort_flag, p.status, 4);
          if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
        if (!ok) break;
        tc_fence_after();
        const int row = m0 + q * 32 + lane;                 // row of the [M x N] problem (= position in the sequence)
        const int ncb = p.N >> 5;                           // 32-column blocks per row
        const int lim = p.rowop_causal ? min(p.N, row + 1) : p.N;                 // valid columns of my row
        const int lim_warp = p.rowop_causal ? min(p.N, m0 + q * 32 + 32) : p.N;   // ... of any row of this warp
        const long long roff = (long long)b1 * p.sC1 + (long long)b2 * p.sC2 + (long long)row * p.ldc;
        // partner exchange area in the unused tail of the operand ring (4 stages of 48 KiB leave 32 KiB)
        float* xch = reinterpret_cast<float*>(smem_gen + 4 * 49152) + ((q * 2 + half) * 32 + lane) * 2;
        float* xch_other = reinterpret_cast<float*>(smem_gen + 4 * 49152) + ((q * 2 + (half ^ 1)) * 32 + lane) * 2;
        auto tcol = [&](int cb) { return tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)accs[cb >> 3] * 256u + (uint32_t)(cb & 7) * 32u; };
        uint32_t v[32];
        if (p.rowop == 1) {
          const float k2 = p.alpha * 1.4426950408889634f;   // base-2 exponentials
          float mx = -INFINITY, sum = 0.f;
          for (int cb = half; cb < ncb; cb += 2) {
            if (cb * 32 >= lim_warp) break;  // warp-uniform: nothing valid from here on
            tmem_ld32(tcol(cb), v);
            tmem_ld_wait();
            float cm = -INFINITY;
#pragma unroll
            for (int j = 0; j < 32; j++) {
              const float x = (cb * 32 + j < lim) ? __uint_as_float(v[j]) * k2 : -INFINITY;
              v[j] = __float_as_uint(x);
              cm = fmaxf(cm, x);
            }
            if (cm > mx) { sum *= fml_exp2_ftz(mx - cm); mx = cm; }
            if (mx != -INFINITY) {
#pragma unroll
              for (int j = 0; j < 32; j++) sum += fml_exp2_ftz(__uint_as_float(v[j]) - mx);
            }
          }
          xch[0] = mx; xch[1] = sum;
          asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory");
          const float om = xch_other[0], os = xch_other[1];
          const float M2 = fmaxf(mx, om);   // finite: column 0 is valid for every row and belongs to one of the two
          const float S2 = (mx == -INFINITY ? 0.f : sum * fml_exp2_ftz(mx - M2)) + (om == -INFINITY ? 0.f : os * fml_exp2_ftz(om - M2));
          const float inv = 1.f / S2;
          for (int cb = half; cb < ncb; cb += 2) {
            float4* dst = reinterpret_cast<float4*>(p.C + roff + cb * 32);
            if (cb * 32 >= lim_warp) {
              if (row < p.M) {
#pragma unroll
                for (int j = 0; j < 8; j++) dst[j] = make_float4(0.f, 0.f, 0.f, 0.f);
              }
              continue;
            }
            tmem_ld32(tcol(cb), v);
            tmem_ld_wait();
            if (row < p.M) {
#pragma unroll
              for (int j = 0; j < 8; j++) {
                float4 o;
                o.x = (cb * 32 + 4 * j + 0 < lim) ? fml_exp2_ftz(__uint_as_float(v[4 * j + 0]) * k2 - M2) * inv : 0.f;
                o.y = (cb * 32 + 4 * j + 1 < lim) ? fml_exp2_ftz(__uint_as_float(v[4 * j + 1]) * k2 - M2) * inv : 0.f;
                o.z = (cb * 32 + 4 * j + 2 < lim) ? fml_exp2_ftz(__uint_as_float(v[4 * j + 2]) * k2 - M2) * inv : 0.f;
                o.w = (cb * 32 + 4 * j + 3 < lim) ? fml_exp2_ftz(__uint_as_float(v[4 * j + 3]) * k2 - M2) * inv : 0.f;
                dst[j] = o;
              }
            }
          }
        } else {
          // dS = alpha * P * (dP - sum_j dP_j P_j); masked P entries are exactly 0
          float dot = 0.f;
          for (int cb = half; cb < ncb; cb += 2) {
            if (cb * 32 >= lim_warp) break;
            tmem_ld32(tcol(cb), v);
            tmem_ld_wait();
            if (row < p.M) {
              const float4* pp = reinterpret_cast<const float4*>(p.rowop_aux + roff + cb * 32);
#pragma unroll
              for (int j = 0; j < 8; j++) {
                const float4 pv = pp[j];
                dot += __uint_as_float(v[4 * j]) * pv.x + __uint_as_float(v[4 * j + 1]) * pv.y +
                       __uint_as_float(v[4 * j + 2]) * pv.z + __uint_as_float(v[4 * j + 3]) * pv.w;
              }
            }
          }
          xch[0] = dot;
          asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory");
          dot += xch_other[0];
          for (int cb = half; cb < ncb; cb += 2) {
            float4* dst = reinterpret_cast<float4*>(p.C + roff + cb * 32);
            if (cb * 32 >= lim_warp) {
              if (row < p.M) {
#pragma unroll
                for (int j = 0; j < 8; j++) dst[j] = make_float4(0.f, 0.f, 0.f, 0.f);
              }
              continue;
            }
            tmem_ld32(tcol(cb), v);
            tmem_ld_wait();
            if (row < p.M) {
              const float4* pp = reinterpret_cast<const float4*>(p.rowop_aux + roff + cb * 32);
#pragma unroll
              for (int j = 0; j < 8; j++) {
                const float4 pv = pp[j];
                dst[j] = make_float4(p.alpha * pv.x * (__uint_as_float(v[4 * j]) - dot),
                                     p.alpha * pv.y * (__uint_as_float(v[4 * j + 1]) - dot),
                                     p.alpha * pv.z * (__uint_as_float(v[4 * j + 2]) - dot),
                                     p.alpha * pv.w * (__uint_as_float(v[4 * j + 3]) - dot));
              }
            }
          }
        }
        // the exchange slots are rewritten only after the partner has read them
        asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0)
          for (int j = 0; j < p.tiles_n; j++) mbar_arrive(tempty_bar(accs[j]));
        it_u += p.tiles_n - 1;  // the unit's remaining n-tiles were consumed here
        continue;
      }
      const int nchunks = (nkb + p.kchunk - 1) / p.kchunk;
     for (int chunk = 0; chunk < nchunks && ok; chunk++) {
      ok = mbar_wait(tfull_bar(acc), acc_ph, abort_flag, p.status, 4);
      if (!ok) break;
      tc_fence_after();
      // 0: whole K in one chunk; 1: first chunk (store partial); 2: middle (add); 3: last (add back, finish)
      const int mode = nchunks == 1 ? 0 : (chunk == 0 ? 1 : (chunk == nchunks - 1 ? 3 : 2));
      float* slab = p.partial + (size_t)blockIdx.x * (BM * 256) + (size_t)(q * 32 + lane) * 32;
      const int row = m0 + q * 32 + lane;
      const long long boff = (long long)b1 * p.sC1 + (long long)b2 * p.sC2 + (long long)row * p.ldc;
      float* crow = p.C + boff;
      float* zrow = p.Z ? p.Z + boff : nullptr;
      const int ncols32 = min(p.BN / 32, (p.N - n0 + 31) / 32);  // 32-column blocks of this tile inside the matrix
      const uint32_t tacc = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * 256u;
      // one 32x32 block of the accumulator, held as one row per thread
      auto process = [&](const int c, uint32_t (&v)[32]) {
        const int col0 = n0 + c * 32;
        if (mode != 0) {
          // this thread owns 32 consecutive floats of the slab per column chunk: [c][row][32]
          float4* sp = reinterpret_cast<float4*>(slab + (size_t)c * (BM * 32));
          if (mode == 1) {
#pragma unroll
            for (int j = 0; j < 8; j++)
              sp[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                                  __uint_as_float(v[4 * j + 3]));
            return;
          }
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const float4 o = sp[j];
            v[4 * j] = __float_as_uint(__uint_as_float(v[4 * j]) + o.x);
            v[4 * j + 1] = __float_as_uint(__uint_as_float(v[4 * j + 1]) + o.y);
            v[4 * j + 2] = __float_as_uint(__uint_as_float(v[4 * j + 2]) + o.z);
            v[4 * j + 3] = __float_as_uint(__uint_as_float(v[4 * j + 3]) + o.w);
          }
          if (mode == 2) {
#pragma unroll
            for (int j = 0; j < 8; j++)
              sp[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                                  __uint_as_float(v[4 * j + 3]));
            return;
          }
        }
        if (p.lstm) {
          // LSTM step: pre-activation = product + input projection; this thread owns batch row `row` and the
          // four gates of hidden units col0/4 .. col0/4 + 7
          if (row < p.M) {
            const int H = p.N >> 2, r0 = col0 >> 2;
            const long long po = (long long)row * p.N + col0, ho = (long long)row * H + r0;
            // all ten loads first: with the loads inside the loop below each one sat behind the previous
            // iteration's store to `gates` (possible alias) and the block cost eight L2 round trips instead of one
            float cp[8];
            float4 xa[8];
            *reinterpret_cast<float4*>(cp) = *reinterpret_cast<const float4*>(p.le.c_prev + ho);
            *reinterpret_cast<float4*>(cp + 4) = *reinterpret_cast<const float4*>(p.le.c_prev + ho + 4);
#pragma unroll
            for (int uu = 0; uu < 8; uu++) xa[uu] = *reinterpret_cast<const float4*>(p.le.addend + po + 4 * uu);
            float cn[8], hn[8];
#pragma unroll
            for (int uu = 0; uu < 8; uu++) {
              const float zf = __uint_as_float(v[4 * uu]) + xa[uu].x, zi = __uint_as_float(v[4 * uu + 1]) + xa[uu].y;
              const float zg = __uint_as_float(v[4 * uu + 2]) + xa[uu].z, zo = __uint_as_float(v[4 * uu + 3]) + xa[uu].w;
              float f, i, g, o;
              if (p.le.fast_math) {
                f = fml_sigmoid_fast(zf); i = fml_sigmoid_fast(zi); g = fml_tanh_fast(zg); o = fml_sigmoid_fast(zo);
              } else {
                f = fml_sigmoid(zf); i = fml_sigmoid(zi); g = fml_tanh_ref(zg); o = fml_sigmoid(zo);
              }
              cn[uu] = f * cp[uu] + i * g;
              hn[uu] = o * (p.le.fast_math ? fml_tanh_fast(cn[uu]) : fml_tanh_ref(cn[uu]));
              *reinterpret_cast<float4*>(p.le.gates + po + 4 * uu) = make_float4(f, i, g, o);
            }
            *reinterpret_cast<float4*>(p.le.c_out + ho) = *reinterpret_cast<float4*>(cn);
            *reinterpret_cast<float4*>(p.le.c_out + ho + 4) = *reinterpret_cast<float4*>(cn + 4);
            *reinterpret_cast<float4*>(p.le.h_out + ho) = *reinterpret_cast<float4*>(hn);
            *reinterpret_cast<float4*>(p.le.h_out + ho + 4) = *reinterpret_cast<float4*>(hn + 4);
          }
          return;
        }
        if (row < p.M) {
          const bool full = (col0 + 32 <= p.N);
          if (full && vec_ok) {
            // The four epilogue warps are the only warps of their schedulers, so every instruction waits out
            // its full latency: the code below keeps branches out of the per-element loops and gives the
            // common plain product (no bias, scale, activation, second output or accumulation) a store-only path.
            float4* cp = reinterpret_cast<float4*>(crow + col0);
            if (plain) {
#pragma unroll
              for (int j = 0; j < 8; j++)
                reinterpret_cast<uint4*>(cp)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              return;
            }
            float o[32];
            if (p.bias) {
#pragma unroll
              for (int j = 0; j < 8; j++) {
                const float4 bz = *reinterpret_cast<const float4*>(p.bias + col0 + 4 * j);
                o[4 * j] = fmaf(__uint_as_float(v[4 * j]), p.alpha, bz.x);
                o[4 * j + 1] = fmaf(__uint_as_float(v[4 * j + 1]), p.alpha, bz.y);
                o[4 * j + 2] = fmaf(__uint_as_float(v[4 * j + 2]), p.alpha, bz.z);
                o[4 * j + 3] = fmaf(__uint_as_float(v[4 * j + 3]), p.alpha, bz.w);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; j++) o[j] = __uint_as_float(v[j]) * p.alpha;
            }
            if (zrow) {
              float4* zp = reinterpret_cast<float4*>(zrow + col0);
#pragma unroll
              for (int j = 0; j < 8; j++) zp[j] = make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
            }
            if (p.act == FML_ACT_RELU) {
#pragma unroll
              for (int j = 0; j < 32; j++) o[j] = o[j] > 0.f ? o[j] : 0.f;
            } else if (p.act != FML_ACT_NONE) {
#pragma unroll
              for (int j = 0; j < 32; j++) o[j] = fml_act_apply_slow(p.act, o[j]);
            }
            if (p.dact_saved) {
              // dLoss/dAct multiply of the layer below: this product is the gradient of that layer's output
              const float4* sp = reinterpret_cast<const float4*>(p.dact_saved + boff + col0);
#pragma unroll
              for (int j = 0; j < 8; j++) {
                const float4 sv = sp[j];
                o[4 * j] *= fml_act_grad_small(p.dact, sv.x);
                o[4 * j + 1] *= fml_act_grad_small(p.dact, sv.y);
                o[4 * j + 2] *= fml_act_grad_small(p.dact, sv.z);
                o[4 * j + 3] *= fml_act_grad_small(p.dact, sv.w);
              }
            }
            if (p.ksplit > 1) {
#pragma unroll
              for (int j = 0; j < 8; j++)  // K split: partial products add up in C
                atomicAdd(cp + j, make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]));
              return;
            }
            if (p.beta != 0.f) {
#pragma unroll
              for (int j = 0; j < 8; j++) {
                const float4 old = cp[j];
                o[4 * j] += old.x; o[4 * j + 1] += old.y; o[4 * j + 2] += old.z; o[4 * j + 3] += old.w;
              }
            }
#pragma unroll
            for (int j = 0; j < 8; j++) cp[j] = make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; j++) {
              const int col = col0 + j;
              if (col < p.N) {
                float o = __uint_as_float(v[j]) * p.alpha + (p.bias ? p.bias[col] : 0.f);
                if (zrow) zrow[col] = o;
                o = fml_act_apply(p.act, o);
                if (p.dact_saved) o *= fml_act_grad_small(p.dact, p.dact_saved[boff + col]);
                if (p.ksplit > 1) { atomicAdd(crow + col, o); continue; }
                if (p.beta != 0.f) o += crow[col];
                crow[col] = o;
              }
            }
          }
        }
      };
      // The eight epilogue warps are the only warps on their schedulers besides the two single-lane roles, so
      // each instruction waits out its full latency; two warps per TMEM lane quarter interleave their blocks.
      for (int c = half; c < ncols32; c += 2) {
        uint32_t v[32];
        tmem_ld32(tacc + (uint32_t)c * 32u, v);
        tmem_ld_wait();
        process(c, v);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR && rank != 0) mbar_arrive_remote(tempty_bar(acc), 0);  // the issuer lives in the leader
        else mbar_arrive(tempty_bar(acc));
      }
      if (++acc == 2) { acc = 0; acc_ph ^= 1; }
     }
    }
  }

  // common tail: everyone arrives (both CTAs of a pair: the peer's barriers and TMEM stay alive
  // until nothing can signal or read them), then the allocating warp frees TMEM
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();
  tc_fence_after();
  if (warp == 1) {
    __syncwarp();
    if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// hi = round-to-nearest tf32 of x, lo = x - hi (exact in fp32); generic 4-level strided source,
// compact destination [b2][b1][rows][ldd].
__global__ void split_tf32_kernel(const float* __restrict__ src, float* __restrict__ hi, float* __restrict__ lo,
                                  int rows, int cols, long long ld, int nb1, int nb2, long long s1, long long s2,
                                  int ldd) {
  const long long total = (long long)nb2 * nb1 * rows * ldd;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    int c = (int)(i % ldd);
    long long r = i / ldd;
    int row = (int)(r % rows);
    long long bb = r / rows;
    int b1 = (int)(bb % nb1), b2 = (int)(bb / nb1);
    float x = 0.f;
    if (c < cols) x = src[(long long)b2 * s2 + (long long)b1 * s1 + (long long)row * ld + c];
    uint32_t h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    float hf = __uint_as_float(h);
    hi[i] = hf;
    lo[i] = x - hf;
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Rank-4 map {cols, rows, nb1, nb2} over a row-major matrix with two batch levels.
int32_t make_tmap(fml_ctx* ctx, const float* base, int64_t cols, int64_t rows, int64_t ld, int64_t nb1, int64_t nb2,
                  int64_t s1, int64_t s2, int box_c, int box_r, bool mn_major, int blocks, CUtensorMap* out) {
  // blocks > 0: rank-5 map {32, rows, cols/32, nb1, nb2} with box {32, 32, blocks, 1, 1} (MN-major, cols % 32 == 0).
  // box_r carries the layout kind in the cache key: negative = MN-major (32B-atom swizzle), offset by the block count
  auto key = std::make_tuple((const void*)base, cols, rows, ld, nb1, nb2, s1, s2, box_c,
                             mn_major ? -(box_r + 1000 * blocks) : box_r);
  auto it = ctx->tmaps.find(key);
  if (it != ctx->tmaps.end()) {
    *out = it->second;
    return FML_OK;
  }
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return fml_fail(ctx, FML_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  // unused batch levels get a harmless, 16-byte-multiple stride
  if (nb1 <= 1) s1 = rows * ld;
  if (nb2 <= 1) s2 = (nb1 <= 1 ? rows * ld : s1 * nb1);
  cuuint64_t dims[5] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)(nb1 < 1 ? 1 : nb1), (cuuint64_t)(nb2 < 1 ? 1 : nb2), 1};
  cuuint64_t strides[4] = {(cuuint64_t)ld * 4, (cuuint64_t)s1 * 4, (cuuint64_t)s2 * 4, 0};
  cuuint32_t box[5] = {(cuuint32_t)box_c, (cuuint32_t)box_r, 1, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  int rank = 4;
  if (blocks > 0) {
    rank = 5;
    dims[0] = 32; dims[1] = (cuuint64_t)rows; dims[2] = (cuuint64_t)(cols / 32);
    dims[3] = (cuuint64_t)(nb1 < 1 ? 1 : nb1); dims[4] = (cuuint64_t)(nb2 < 1 ? 1 : nb2);
    strides[0] = (cuuint64_t)ld * 4; strides[1] = 128; strides[2] = (cuuint64_t)s1 * 4; strides[3] = (cuuint64_t)s2 * 4;
    box[0] = 32; box[1] = 32; box[2] = (cuuint32_t)blocks; box[3] = 1; box[4] = 1;
  }
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, rank, const_cast<float*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char msg[256];
    snprintf(msg, sizeof msg, "cuTensorMapEncodeTiled failed (%d): cols=%lld rows=%lld ld=%lld nb=(%lld,%lld) s=(%lld,%lld) box=(%d,%d)",
             (int)r, (long long)cols, (long long)rows, (long long)ld, (long long)nb1, (long long)nb2, (long long)s1,
             (long long)s2, box_c, box_r);
    return fml_fail(ctx, FML_ERR_CUDA, msg);
  }
  if (ctx->tmaps.size() > 4096) ctx->tmaps.clear();
  ctx->tmaps[key] = *out;
  return FML_OK;
}

bool splitk_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("FML_GEMM_SPLITK");  // diagnostics: 0 disables the K split
    v = e ? atoi(e) : 1;
  }
  return v != 0;
}

uint32_t make_idesc(int M, int BN, int a_mn, int b_mn) {
  uint32_t d = 0;
  d |= 1u << 4;                    // accumulator format F32
  d |= 2u << 7;                    // A format TF32
  d |= 2u << 10;                   // B format TF32
  d |= (uint32_t)(a_mn & 1) << 15; // A major-ness (0 = K, 1 = MN)
  d |= (uint32_t)(b_mn & 1) << 16; // B major-ness
  d |= (uint32_t)(BN >> 3) << 17;  // N / 8
  d |= (uint32_t)(M >> 4) << 24;   // M / 16 (256 spans both CTAs of a pair)
  return d;
}

}  // namespace

namespace {
// One CTA waits on an mbarrier that nothing ever arrives at, with the same bounded wait every pipeline role of the
// tensor-core kernels uses, and must come back with the error code instead of hanging.
__global__ void wait_timeout_selftest_kernel(int* status, unsigned long long limit_ns) {
  __shared__ alignas(8) unsigned long long mbar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&mbar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_wait_limit(smem_u32(&mbar), 0, &abort_flag, status, 99, limit_ns);
  }
}
}  // namespace

extern "C" int32_t fml_selftest_wait_timeout(fml_ctx* ctx, int32_t limit_us) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, ctx && limit_us > 0 && limit_us <= 1000000, "fml_selftest_wait_timeout: the limit must be 1 .. 1000000 us");
  wait_timeout_selftest_kernel<<<1, 32, 0, ctx->stream>>>(ctx->d_status, (unsigned long long)limit_us * 1000ull);
  FML_LAUNCH_CHECK(ctx, "wait_timeout_selftest_kernel");
  return FML_OK;
}

int32_t fml_tc_make_tmap(fml_ctx* ctx, const float* base, int64_t cols, int64_t rows, int64_t ld, int64_t nb1, int64_t nb2,
                         int64_t s1, int64_t s2, int box_c, int box_r, bool mn_major, int blocks, CUtensorMap* out) {
  return make_tmap(ctx, base, cols, rows, ld, nb1, nb2, s1, s2, box_c, box_r, mn_major, blocks, out);
}

bool fml_gemm_tc_eligible(const fml_gemm_desc* d) {
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!al16(d->A) || !al16(d->B)) return false;
  if ((d->lda & 3) || (d->ldb & 3)) return false;
  if (d->batch1 > 1 && ((d->sA1 & 3) || (d->sB1 & 3))) return false;
  if (d->batch2 > 1 && ((d->sA2 & 3) || (d->sB2 & 3))) return false;
  return true;
}

int32_t fml_gemm_tc(fml_ctx* ctx, const fml_gemm_desc* d, int precision, const fml_lstm_epilogue* lstm) {
  FML_ONCE_PER_DEVICE(ctx, {
    FML_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<false>::SMEM_BYTES));
    FML_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<true>::SMEM_BYTES));
  });
  const int nb1 = d->batch1 < 1 ? 1 : d->batch1, nb2 = d->batch2 < 1 ? 1 : d->batch2;
  // pair mode (256 x 256 tiles over two CTAs) when the problem has enough such tiles to occupy the
  // machine; FML_GEMM_PAIR=0/1 forces the choice (diagnostics)
  const long long pair_tiles = (long long)((d->M + 255) / 256) * ((d->N + 255) / 256) * nb1 * nb2;
  bool pair = d->M > 128 && d->N > 128 && pair_tiles >= ctx->sm_count / 4;
  // A plain TF32 product with few output tiles but a long K (weight gradients: K = all tokens of the batch) can
  // still fill the machine with 256 x 256 pair tiles if its K range is divided over several pairs; narrow single
  // tiles ran such products at a third of the rate (1024 x 1024 x 16384: 180 TFLOP/s with 128 x 64 tiles).
  const bool splittable = precision == FML_PREC_TF32 && !d->rowop && nb1 * nb2 == 1 && !d->bias && !d->preact &&
                          d->act == FML_ACT_NONE && !lstm && !d->dact_saved && splitk_enabled();
  if (!pair && splittable && d->M > 128 && d->N > 128 && pair_tiles * ((d->K + BK - 1) / BK / 8) >= ctx->sm_count / 4) pair = true;
  if (d->rowop) pair = false;  // a row block (128 rows x up to 512 columns) lives in ONE CTA's tensor memory
  {
    static int force = -2;
    if (force == -2) {
      const char* e = getenv("FML_GEMM_PAIR");
      force = e ? atoi(e) : -1;
    }
    if (force >= 0 && !d->rowop) pair = force != 0;
  }
  const int tile_m = pair ? 2 * BM : BM;
  const int tiles_m = (d->M + tile_m - 1) / tile_m;
  // widest tile that still gives every SM work
  int BN = 64;
  if (pair || d->rowop) BN = 256;
  else for (int bn : {256, 128, 64}) {
    long long tiles = (long long)tiles_m * ((d->N + bn - 1) / bn) * nb1 * nb2;
    if (d->N > bn / 2 && tiles >= ctx->sm_count) { BN = bn; break; }
  }
  if (BN == 64 && !pair && !d->rowop) {
    // small problem: nothing fills the machine; prefer the tile that wastes least of N
    BN = d->N > 128 ? (d->N > 192 ? 256 : 128) : (d->N > 64 ? 128 : 64);
    long long t256 = (long long)tiles_m * ((d->N + 255) / 256) * nb1 * nb2;
    if (BN == 256 && t256 < ctx->sm_count / 2) BN = 128;
    long long t128 = (long long)tiles_m * ((d->N + 127) / 128) * nb1 * nb2;
    if (BN == 128 && t128 < ctx->sm_count / 2 && d->N > 64) BN = 64;
  }
  const int tiles_n = (d->N + BN - 1) / BN;
  const int a_mn = d->transA ? 1 : 0;  // stored [K x M]: M contiguous
  const int b_mn = d->transB ? 0 : 1;  // stored [K x N]: N contiguous

  const float* A = d->A;
  const float* B = d->B;
  const float *Alo = nullptr, *Blo = nullptr;
  size_t split_bytes = 0;
  int64_t lda = d->lda, ldb = d->ldb, sA1 = d->sA1, sA2 = d->sA2, sB1 = d->sB1, sB2 = d->sB2;
  const int64_t a_rows = d->transA ? d->K : d->M, a_cols = d->transA ? d->M : d->K;
  const int64_t b_rows = d->transB ? d->N : d->K, b_cols = d->transB ? d->K : d->N;
  if (precision == FML_PREC_3XTF32) {
    const int64_t a_ldd = (a_cols + 3) & ~3ll, b_ldd = (b_cols + 3) & ~3ll;
    const size_t a_n = (size_t)nb1 * nb2 * a_rows * a_ldd, b_n = (size_t)nb1 * nb2 * b_rows * b_ldd;
    split_bytes = (2 * a_n + 2 * b_n) * sizeof(float);
    // room for the chunk slabs too, so the arena is not reallocated after the split kernels are queued
    int32_t rc = fml_ensure_workspace(ctx, split_bytes + 1024 + (size_t)ctx->sm_count * BM * 256 * sizeof(float));
    if (rc) return rc;
    float* w = reinterpret_cast<float*>(ctx->ws);
    float *Ahi = w, *Al = w + a_n, *Bhi = w + 2 * a_n, *Bl = w + 2 * a_n + b_n;
    const int threads = 256;
    auto blocks = [&](size_t n) { return (int)std::min<size_t>((n + threads - 1) / threads, (size_t)ctx->sm_count * 16); };
    split_tf32_kernel<<<blocks(a_n), threads, 0, ctx->stream>>>(d->A, Ahi, Al, (int)a_rows, (int)a_cols, d->lda, nb1, nb2,
                                                                d->sA1, d->sA2, (int)a_ldd);
    split_tf32_kernel<<<blocks(b_n), threads, 0, ctx->stream>>>(d->B, Bhi, Bl, (int)b_rows, (int)b_cols, d->ldb, nb1, nb2,
                                                                d->sB1, d->sB2, (int)b_ldd);
    FML_LAUNCH_CHECK(ctx, "split_tf32_kernel");
    A = Ahi; Alo = Al; B = Bhi; Blo = Bl;
    lda = a_ldd; ldb = b_ldd;
    sA1 = a_rows * a_ldd; sA2 = sA1 * nb1;
    sB1 = b_rows * b_ldd; sB2 = sB1 * nb1;
  }

  CUtensorMap tmA, tmB, tmAlo, tmBlo;
  int32_t rc;
  const int a_blk = (a_mn && a_cols % 32 == 0) ? BM / 32 : 0;
  const int b_blk = (b_mn && b_cols % 32 == 0) ? (pair ? BN / 2 : BN) / 32 : 0;
  const int a_box_c = 32, a_box_r = a_mn ? 32 : BM;
  const int b_box_c = 32, b_box_r = b_mn ? 32 : (pair ? BN / 2 : BN);
  if ((rc = make_tmap(ctx, A, a_cols, a_rows, lda, nb1, nb2, sA1, sA2, a_box_c, a_box_r, a_mn, a_blk, &tmA))) return rc;
  if ((rc = make_tmap(ctx, B, b_cols, b_rows, ldb, nb1, nb2, sB1, sB2, b_box_c, b_box_r, b_mn, b_blk, &tmB))) return rc;
  if (Alo) {
    if ((rc = make_tmap(ctx, Alo, a_cols, a_rows, lda, nb1, nb2, sA1, sA2, a_box_c, a_box_r, a_mn, a_blk, &tmAlo))) return rc;
    if ((rc = make_tmap(ctx, Blo, b_cols, b_rows, ldb, nb1, nb2, sB1, sB2, b_box_c, b_box_r, b_mn, b_blk, &tmBlo))) return rc;
  } else {
    tmAlo = tmA;
    tmBlo = tmB;
  }

  TcParams p;
  p.rowop = d->rowop; p.rowop_causal = d->rowop_causal; p.rowop_aux = d->rowop_aux;
  p.dact_saved = d->dact_saved;
  p.dact = d->dact;
  p.lstm = lstm ? 1 : 0;
  if (lstm) {
    p.le = *lstm;
  } else {
    p.le = fml_lstm_epilogue{nullptr, nullptr, nullptr, nullptr, nullptr, 0};
  }
  p.M = d->M; p.N = d->N; p.K = d->K;
  p.tiles_m = tiles_m; p.tiles_n = tiles_n; p.nb1 = nb1; p.nb2 = nb2;
  p.BN = BN; p.a_mn = a_mn; p.b_mn = b_mn; p.a_blk = a_blk; p.b_blk = b_blk;
  p.nseg = (precision == FML_PREC_3XTF32) ? 3 : 1;
  {
    // A panel of a group (group_m * tile_m rows x K) should occupy about half of the 126 MB L2.  Measured at
    // 8192^3 with groups of 4096 rows (128 MB panels): 2.6 GB read from DRAM per launch against 0.5 GB algorithmic.
    const long long rows = (64ll << 20) / (4ll * std::max(d->K, 1));
    int g = (int)std::max<long long>(1, std::min<long long>(rows / tile_m, 32));
    static int force = -2;
    if (force == -2) {
      const char* e = getenv("FML_GEMM_GROUP_M");  // diagnostics
      force = e ? atoi(e) : -1;
    }
    p.group_m = force > 0 ? force : g;
  }
  p.stage_bytes = A_STAGE_BYTES + (pair ? BN / 2 : BN) * BK * 4;
  p.nstages = std::min((int)Cfg<false>::MAX_STAGES, (int)Cfg<false>::RING_BYTES / p.stage_bytes);
  p.kblocks = (d->K + BK - 1) / BK;
  p.kchunk = (precision == FML_PREC_3XTF32 ? 1024 : 8192) / BK;
  if (p.kblocks <= p.kchunk + p.kchunk / 4 || d->rowop) p.kchunk = p.kblocks;  // not worth a second chunk for a short tail
  p.partial = nullptr;
  p.ksplit = 1;
  p.kb_per_split = p.kblocks;
  {
    // K split for plain TF32 products whose tiles occupy less than ~60 % of the SMs
    const long long tiles_all = (long long)tiles_m * tiles_n * nb1 * nb2;
    const long long ctas = tiles_all * (pair ? 2 : 1);
    if (splittable && ctas * 5 < (long long)ctx->sm_count * 3 && p.kblocks >= 8) {
      int want = (int)(ctx->sm_count / ctas);                 // CTAs available per tile
      int maxs = p.kblocks / 4;                               // at least 128 k per split
      int ks = std::max(1, std::min(want, maxs));
      if (ks > 1) {
        p.kb_per_split = (p.kblocks + ks - 1) / ks;
        p.ksplit = (p.kblocks + p.kb_per_split - 1) / p.kb_per_split;
        if (d->beta == 0.f)
          FML_CUDA(ctx, cudaMemset2DAsync(d->C, (size_t)d->ldc * 4, 0, (size_t)d->N * 4, (size_t)d->M, ctx->stream));
      }
    } else if (splittable && p.kblocks >= 64 && (long long)d->M * d->N <= (4ll << 20)) {
      // Partial single wave (a weight gradient with 48 pair tiles on 74 pairs leaves a third of the machine idle
      // for the whole K loop): a small K split that makes the work units fill whole waves.  cost = waves / split.
      const long long slots = pair ? ctx->sm_count / 2 : ctx->sm_count;
      if (tiles_all < slots) {
        int best = 1;
        double best_cost = 1.0;
        for (int ks = 2; ks <= 6; ks++) {
          const double cost = (double)((tiles_all * ks + slots - 1) / slots) / ks * (1.0 + 0.03 * (ks - 1));
          if (cost < best_cost * 0.85) { best = ks; best_cost = cost; }
        }
        if (best > 1) {
          p.kb_per_split = (p.kblocks + best - 1) / best;
          p.ksplit = (p.kblocks + p.kb_per_split - 1) / p.kb_per_split;
          if (d->beta == 0.f)
            FML_CUDA(ctx, cudaMemset2DAsync(d->C, (size_t)d->ldc * 4, 0, (size_t)d->N * 4, (size_t)d->M, ctx->stream));
        }
      }
    }
  }
  p.C = d->C; p.Z = d->preact; p.bias = d->bias;
  p.ldc = d->ldc; p.sC1 = d->sC1; p.sC2 = d->sC2;
  p.act = d->act; p.alpha = d->alpha; p.beta = d->beta;
  p.status = ctx->d_status;
  p.idesc = make_idesc(tile_m, BN, a_mn, b_mn);
  p.debug = 0;
#ifdef FML_GEMM_DIAGNOSTICS  // a build with -DFML_GEMM_DIAGNOSTICS can skip the loads or the MMAs (FML_GEMM_DEBUG=1|2) to time the other half
  {
    static int dbg = -1;
    if (dbg < 0) {
      const char* e = getenv("FML_GEMM_DEBUG");
      dbg = e ? atoi(e) : 0;
    }
    p.debug = dbg;
  }
#endif
  const long long num_tiles = (long long)tiles_m * tiles_n * nb1 * nb2 * p.ksplit;  // work units
  // SMs this persistent launch may occupy: all of them, less the ones set aside for a collective that runs beside it
  const int grid_sms = std::max(2, ctx->sm_count - ctx->sm_reserve);
  if (p.kchunk < p.kb_per_split) {
    // slabs live behind whatever the 3xTF32 split already placed in the arena
    const size_t grid_ctas = pair ? 2 * (size_t)std::min<long long>(num_tiles, grid_sms / 2)
                                  : (size_t)std::min<long long>(num_tiles, grid_sms);
    const size_t slab_bytes = grid_ctas * BM * 256 * sizeof(float);
    const size_t off = (split_bytes + 1023) & ~(size_t)1023;
    // with a split queued on the stream the arena must stay where it is (it was sized for the slabs above)
    if ((rc = split_bytes ? fml_ensure_workspace_keep(ctx, off + slab_bytes) : fml_ensure_workspace(ctx, off + slab_bytes))) return rc;
    p.partial = reinterpret_cast<float*>(ctx->ws + off);
  }
  static int pdl = -1;
  if (pdl < 0) {
    const char* e = getenv("FML_GEMM_PDL");
    pdl = e ? atoi(e) : 1;
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (pdl) {  // this kernel's prologue may overlap the tail of the kernel queued before it
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    na++;
  }
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.stream = ctx->stream;
  cfg.attrs = attr;
  if (pair) {
    const int clusters = (int)std::min<long long>(num_tiles, grid_sms / 2);
    cfg.gridDim = dim3(2 * clusters);
    cfg.dynamicSmemBytes = Cfg<true>::SMEM_BYTES;
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 2;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    na++;
    cfg.numAttrs = na;
    FML_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_tc_kernel<true>, tmA, tmB, tmAlo, tmBlo, p));
  } else {
    const int grid = (int)std::min<long long>(d->rowop ? num_tiles / tiles_n : num_tiles, grid_sms);
    cfg.gridDim = dim3(grid);
    cfg.dynamicSmemBytes = Cfg<false>::SMEM_BYTES;
    cfg.numAttrs = na;
    FML_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_tc_kernel<false>, tmA, tmB, tmAlo, tmBlo, p));
  }
  FML_LAUNCH_CHECK(ctx, "gemm_tc_kernel");
  ctx->last_gemm_path = 1;
  ctx->last_gemm_tile[0] = pair ? 2 : 1;
  ctx->last_gemm_tile[1] = BN;
  ctx->last_gemm_tile[2] = p.ksplit;
  ctx->last_gemm_tile[3] = (p.kb_per_split + p.kchunk - 1) / p.kchunk;
  return FML_OK;
}
