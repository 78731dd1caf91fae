// Tensor-core convolution for narrow layers (at most 64 output channels): implicit GEMM on CTA pairs
// with the whole filter resident in shared memory.
//
// Rows of the GEMM are output pixels, N is the output-channel count (<= 64), K runs over
// (kh, kw, 32-channel block). With N = 64 a tcgen05.mma is too small to keep the tensor pipe busy from a
// single-CTA instruction stream, so two CTAs form a cluster and one instruction (cta_group::2, M = 256)
// covers 256 pixels: 128 per CTA (a tile of 8 x 16 output pixels), two such tiles per pair. Per CTA:
//   * the filter half this CTA contributes to the pair's B operand (N/2 channels x all of K, repacked and,
//     in 3xTF32 mode, pre-split into hi / lo once by conv2d_prepare_filter) is loaded ONCE and stays in shared
//     memory for the life of the persistent CTA -- it is not re-streamed per tile;
//   * activations arrive NHWC through a ring of stages. A stage is the input slab under ONE filter column kw
//     (and up to two 32-channel blocks): 8 pixels wide, 16 + KH - 1 pixels high, fetched by one 5-D TMA box
//     {32 c, 8 w, 16 + KH - 1 h, 2 channel blocks, 1 n} at (0, ow0 + kw - pad, oh0 - pad, cb, n). Its rows are
//     (h, w) pixels, 8 per image row, so the A operand of filter tap (kh, kw) is the 128 rows that start kh
//     image rows = kh * 1024 bytes into the slab: the KH taps of a column share one load, and the input crosses
//     the L2 -> shared-memory path KW times instead of KH * KW times (that path, not the tensor pipe, bounded a
//     version with one load per tap). Out-of-range coordinates are zero-filled by the TMA unit, which is the
//     zero padding. Two threads take turns issuing these loads (even / odd stages);
//   * four threads (two in 3xTF32 mode) of the even CTA issue the MMAs, each its share of the k-steps of every
//     k-block into its own TMEM accumulators (one thread alone cannot issue N = 64 instructions as fast as the
//     pipe retires them); the epilogue adds the accumulators;
//   * 3xTF32 mode: eight split warps (two groups on alternate k-blocks) turn the landed rows into
//     hi = tf32(x) and lo = tf32(x - hi) halves in TMEM (the MMAs read A from TMEM, B_hi / B_lo from the
//     resident filter) and run lo*hi + hi*lo + hi*hi;
//     accumulation is cut into chunks whose partial sums the epilogue adds in registers with round-to-nearest
//     (the tensor core adds into its accumulator with round-toward-zero);
//   * the epilogue applies bias / ReLU and writes either NHWC (each thread 128 contiguous bytes of its pixel:
//     the layout the next convolution of a stack reads without any transpose) or NCHW.
// No TMA multicast is used. Every mbarrier wait is bounded (see tc_common.cuh).
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "contract.cuh"
#include "tc_common.cuh"

namespace b200 {
using namespace tc;
namespace {

constexpr int BM = 128;                     // output pixels per CTA and tile: 8 wide x 16 high
constexpr int TW = 8, TH = 16;
constexpr int BK = 32;                      // channels per k-block = one 128-byte swizzle row
constexpr int UMMA_K = 8;
constexpr int A_STAGE_BYTES = BM * BK * 4;  // 16 KiB
constexpr int kMaxStages = 8;
constexpr int kSlots = 4;                   // TMEM slots for A's hi / lo halves (3xTF32), 64 columns each
constexpr int kAccCols = 64;                // columns per accumulator
constexpr int kMaxChunkKb = 20;             // 3xTF32: most k-blocks per accumulation chunk (60 products per accumulator)
constexpr int kBarrierBytes = 512;
constexpr int kMaxDynamicSmem = 227 * 1024 - 1024;  // the rest of the 227 KiB is the kernel's static shared memory

struct ConvPairParams {
  int KH, KW, pad_h, pad_w;
  int OH, OW;
  int slab_bytes;              // one channel block of a stage: (16 + KH - 1) image rows x 8 pixels x 128 bytes
  int tiles_w, tiles_per_img;  // 8 x 16 pixel tiles per row of tiles / per image
  int cblocks, num_kb;
  int chunk_kb;           // 3xTF32: k-blocks summed in one accumulator before the epilogue warps take it over
  int kbs;                // 32-channel blocks per stage: 2, or 1 when the input has at most 32 channels
  int groups;             // stages per filter column
  int stages_per_tile;    // KW * groups
  int64_t total_tiles;    // images * tiles_per_img
  int64_t num_tiles;      // pairs of tiles
  int bn;                // output channels rounded up to a multiple of 16 (the instruction's N)
  int M;                 // output channels
  int stages;
  int b_kb_bytes;        // bytes of resident filter per k-block and CTA
  int y_nhwc;
  int epilogue;
  int vec8;              // NHWC output rows can be written with 32-byte stores
  const float *bias;
  float *Y;
  unsigned *status;
};

__device__ __forceinline__ void st_global_v8(float *p, const float *v) {
  asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
               : "memory");
}

template <bool SPLIT3>
struct PairCfg {
  static constexpr int kEpilogueWarp0 = 4, kEpilogueWarps = 8;
  static constexpr int kSplitWarp0 = kEpilogueWarp0 + kEpilogueWarps, kSplitWarps = SPLIT3 ? 8 : 0;
  // Threads that issue MMAs (even CTA): four, in warps of their own. One thread issues a tcgen05.mma every ~55
  // cycles at best, and every barrier wait in between costs it ~200 more (measured), while an N = 64 pair
  // instruction occupies the tensor pipe for ~53 cycles with A in shared memory and ~36 with A in TMEM.
  //   TF32:   issuer i takes k-step i of every k-block into two accumulators of its own (all 512 TMEM columns);
  //           it waits and commits once per stage.
  //   3xTF32: A's hi / lo halves come through four 64-column TMEM slots, one k-block each. Issuer i owns slot i,
  //           i.e. the k-blocks whose running number is i modulo 4, and issues all twelve products of such a
  //           k-block (one wait and one commit per twelve MMAs) into its one accumulator; the other half of TMEM
  //           holds the slots, so an issuer waits for the epilogue warps at every chunk boundary.
  static constexpr int kIssuers = 4;
  static constexpr int kBufs = SPLIT3 ? 1 : 2;
  static constexpr int kStepsPerIssuer = SPLIT3 ? BK / UMMA_K : (BK / UMMA_K) / kIssuers;
  static constexpr int kExtraIssuerWarp0 = kSplitWarp0 + kSplitWarps;
  // 3xTF32 runs three times longer per stage: one TMA producer is enough there and warp 3 issues MMAs instead
  static constexpr int kProducers = SPLIT3 ? 1 : 2;
  static constexpr int kLowIssuers = 4 - kProducers;  // issuers among warps 1..3
  static constexpr int kThreads = 32 * (kExtraIssuerWarp0 + kIssuers - kLowIssuers);
  static constexpr int kTmemCols = 512;  // kBufs accumulators per issuer (+ 4 A slots in 3xTF32 mode)
  static constexpr int kSlotCol0 = 4 * kAccCols;
};

// Round an fp32 value to TF32 precision (nearest, ties away from zero: what cvt.rna.tf32.f32 computes) with an
// integer add and a mask; the split warps convert 64 values per thread and k-block, and this form measured 6 %
// faster for the whole kernel than the conversion instruction.
__device__ __forceinline__ uint32_t split_hi(float x) { return (__float_as_uint(x) + 0x1000u) & 0xffffe000u; }

// 3xTF32: does issuer i (owner of the k-blocks whose running number is i modulo 4) own a k-block in [lo, hi)?
__device__ __forceinline__ bool chunk_has(int i, int64_t lo, int64_t hi) { return lo + ((i - (int)(lo & 3)) & 3) < hi; }

template <bool SPLIT3>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg<SPLIT3>::kThreads, 1)
conv_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_wlo, const ConvPairParams p) {
  using C = PairCfg<SPLIT3>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int b_bytes = p.num_kb * p.b_kb_bytes;  // resident filter, a multiple of 1024
  const int stage_bytes = p.kbs * p.slab_bytes;
  uint8_t *stages = smem + b_bytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(stages + (size_t)p.stages * stage_bytes);
  // full[8] empty[8] split[4] slotfree[4] tfull[8] tempty[8] bfull
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * kMaxStages;
  const uint32_t bar_split = bar_empty + 8 * kMaxStages;
  const uint32_t bar_slotfree = bar_split + 8 * kSlots;
  const uint32_t bar_tfull = bar_slotfree + 8 * kSlots;
  const uint32_t bar_tempty = bar_tfull + 8 * 8;
  const uint32_t bar_bfull = bar_tempty + 8 * 8;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ __align__(16) float s_bias[kAccCols];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t stage_base = smem_base + (uint32_t)b_bytes;
  const uint32_t rank = cluster_ctarank();
  const int64_t pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int kStages = p.stages;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      // stage release: the issuing threads' commits (TF32) or this CTA's split warps (3xTF32)
      mbar_init(bar_empty + 8 * s, SPLIT3 ? C::kSplitWarps : C::kIssuers);
    }
    for (int t = 0; t < kSlots; ++t) {
      mbar_init(bar_split + 8 * t, 2 * 4);  // one arrival per split warp of one group, both CTAs
      mbar_init(bar_slotfree + 8 * t, 1);    // the commit of the issuing thread that owns the slot
    }
    for (int a = 0; a < C::kBufs * C::kIssuers; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 2 * C::kEpilogueWarps);  // one arrival per epilogue warp of both CTAs
    }
    mbar_init(bar_bfull, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < kAccCols) s_bias[threadIdx.x] = (p.bias && (int)threadIdx.x < p.M) ? __ldg(p.bias + threadIdx.x) : 0.f;
  if (warp == 3) {
    tmem_alloc_pair(smem_u32(&s_tmem_base), C::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int *abort_flag = &s_abort;

  if (warp == 0 || (warp == 3 && C::kProducers == 2)) {
    // ------------------------------- TMA producers (both CTAs) -------------------------------
    // With two threads per CTA (TF32 mode), producer j (warp 0: j = 0, warp 3: j = 1) loads the stages whose running
    // number is congruent to j modulo 2. A stage is one filter column and p.kbs channel blocks, one TMA instruction.
    if (lane == 0) {
      const int j = warp == 0 ? 0 : 1;
      if (j == 0) {
        // The filter half of this CTA, once. The even CTA's barrier counts the bytes of both CTAs (the issuing
        // threads live there): it posts the expectation, the partner's loads complete on it remotely.
        const uint32_t bfull = rank == 0 ? bar_bfull : map_to_cta(bar_bfull, 0);
        if (rank == 0) mbar_expect_tx(bar_bfull, 2u * (uint32_t)b_bytes);
        const int half_rows = p.bn / 2;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          const uint32_t dst = smem_base + (uint32_t)(kb * p.b_kb_bytes);
          if (rank == 0) {
            tma_load_4d(dst, &map_w, bfull, kb * BK, 0, 0, 0);
            if (SPLIT3) tma_load_4d(dst + half_rows * 128, &map_wlo, bfull, kb * BK, 0, 0, 0);
          } else {
            tma_load_4d_pair(dst, &map_w, bfull, kb * BK, half_rows, 0, 0);
            if (SPLIT3) tma_load_4d_pair(dst + half_rows * 128, &map_wlo, bfull, kb * BK, half_rows, 0, 0);
          }
        }
      }
      bool ok = true;
      const uint32_t full_pair0 = map_to_cta(bar_full, 0);
      int64_t g = 0;  // running stage number of this CTA
      for (int64_t tile = pair; tile < p.num_tiles && ok; tile += num_pairs) {
        // this CTA's 8 x 16 tile of output pixels, decomposed once per tile
        const int64_t ct = 2 * tile + (int64_t)rank;
        const int img = (int)(ct / p.tiles_per_img);
        const int rem = (int)(ct - (int64_t)img * p.tiles_per_img);
        const int ty = rem / p.tiles_w;
        const int y0 = ty * TH - p.pad_h, x0 = (rem - ty * p.tiles_w) * TW - p.pad_w;
        int kw = 0, grp = 0;
        for (int st = 0; st < p.stages_per_tile; ++st, ++g) {
          if (C::kProducers == 1 || (g & 1) == j) {
            const int s = (int)(g % kStages);
            const uint32_t ph = (uint32_t)((g / kStages) & 1);
            if (!(ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 1u))) break;
            const uint32_t dst = stage_base + (uint32_t)(s * stage_bytes);
            if (SPLIT3) {
              // each CTA's split warps consume its own stage: local barrier, local bytes
              mbar_expect_tx(bar_full + 8 * s, (uint32_t)stage_bytes);
              tma_load_5d(dst, &map_x, bar_full + 8 * s, 0, x0 + kw, y0, grp * 2, img);
            } else if (rank == 0) {
              // the issuing threads (even CTA) consume both CTAs' stages: one barrier there for both
              mbar_expect_tx(bar_full + 8 * s, 2u * (uint32_t)stage_bytes);
              tma_load_5d(dst, &map_x, bar_full + 8 * s, 0, x0 + kw, y0, grp * 2, img);
            } else {
              tma_load_5d_pair(dst, &map_x, full_pair0 + 8 * s, 0, x0 + kw, y0, grp * 2, img);
            }
          }
          if (++grp == p.groups) { grp = 0; ++kw; }
        }
      }
    }
  } else if (warp <= 3 || warp >= C::kExtraIssuerWarp0) {
    // ------------------------------- MMA issuers (even CTA) -------------------------------
    // Issuer i runs its k-steps of every k-block into its own accumulators (buffers kBufs * i ...).
    if (lane == 0 && rank == 0) {
      const int i = warp <= 3 ? warp - 1 : C::kLowIssuers + (warp - C::kExtraIssuerWarp0);
      constexpr int kSteps = C::kStepsPerIssuer;
      const uint32_t idesc = make_idesc_pair(p.bn, false);
      constexpr uint32_t kStep = (UMMA_K * 4) >> 4;  // 32 bytes inside the swizzle row
      const uint32_t step0 = SPLIT3 ? 0u : (uint32_t)i * kStep;  // TF32: this issuer's k-step of every k-block
      const uint64_t a_desc0 = make_smem_desc(stage_base, 16, 1024, kLayoutSw128) + step0;
      const uint64_t b_desc0 = make_smem_desc(smem_base, 16, 1024, kLayoutSw128) + step0;
      const uint32_t b_kb16 = (uint32_t)p.b_kb_bytes >> 4;
      const uint32_t b_lo16 = (uint32_t)(p.bn / 2 * 128) >> 4;
      const uint32_t stage16 = (uint32_t)stage_bytes >> 4;
      bool ok = mbar_wait(bar_bfull, 0, abort_flag, p.status, 64u);
      tc_fence_after();
      int s = 0, buf = 0;
      uint32_t ph = 0, buf_ph = 0;
      int64_t nrun = 0;  // 3xTF32: running k-block number of this pair (slot nrun % 4, owned by issuer nrun % 4)
      const uint32_t slab16 = (uint32_t)p.slab_bytes >> 4;
      const uint32_t a_t = tmem_base + C::kSlotCol0 + (uint32_t)i * 64;  // 3xTF32: this issuer's slot (hi, then lo)
      for (int64_t tile = pair; tile < p.num_tiles && ok; tile += num_pairs) {
        // K order of a tile: filter column kw, channel-block group, channel block q, filter row kh -- the order
        // in which the slabs arrive. `n` counts the tile's k-blocks; 3xTF32 hands its accumulator to the epilogue
        // warps every p.chunk_kb of them (if it received anything in the chunk).
        int n = 0, kw = 0, grp = 0;
        int a = C::kBufs * i + buf;
        uint32_t d_tmem = tmem_base + (uint32_t)(a * kAccCols);
        bool active = !SPLIT3 || chunk_has(i, nrun, nrun + (p.chunk_kb < p.num_kb ? p.chunk_kb : p.num_kb));
        uint32_t fresh = 1;  // 3xTF32: the accumulator has not received a product of this chunk yet
        if (active) {
          if (!(ok = mbar_wait(bar_tempty + 8 * a, buf_ph ^ 1, abort_flag, p.status, 2u))) break;
          tc_fence_after();
        }
        for (int st = 0; st < p.stages_per_tile && ok; ++st) {
          const int nkb = p.cblocks - grp * 2 < p.kbs ? p.cblocks - grp * 2 : p.kbs;  // valid channel blocks here
          if (!SPLIT3) {
            if (!(ok = mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 4u))) break;
            tc_fence_after();
          }
          for (int q = 0; q < nkb && ok; ++q) {
            for (int kh = 0; kh < p.KH; ++kh, ++n) {
              const int kb = (kh * p.KW + kw) * p.cblocks + grp * 2 + q;  // this k-block's slice of the filter
              const uint64_t b_d = b_desc0 + (uint32_t)kb * b_kb16;
              if (SPLIT3) {
                if (n && n % p.chunk_kb == 0) {
                  // chunk boundary: publish the accumulator, take it back once the epilogue warps have read it
                  if (active) {
                    umma_commit_pair_both(bar_tfull + 8 * a, 3);
                    buf_ph ^= 1;
                  }
                  const int64_t c0 = nrun, left = p.num_kb - n;
                  active = chunk_has(i, c0, c0 + (p.chunk_kb < left ? p.chunk_kb : left));
                  fresh = 1;
                  if (active) {
                    if (!(ok = mbar_wait(bar_tempty + 8 * a, buf_ph ^ 1, abort_flag, p.status, 2u))) break;
                    tc_fence_after();
                  }
                }
                if ((int)(nrun & 3) == i) {
                  if (!(ok = mbar_wait(bar_split + 8 * i, (uint32_t)(nrun >> 2) & 1u, abort_flag, p.status, 4u))) break;
                  tc_fence_after();
#pragma unroll
                  for (int j = 0; j < kSteps; ++j) {
                    umma_tf32_ts_pair(d_tmem, a_t + j * UMMA_K + 32, b_d + j * kStep, idesc, j > 0 ? 1u : fresh ^ 1u);  // lo * hi
                    umma_tf32_ts_pair(d_tmem, a_t + j * UMMA_K, b_d + b_lo16 + j * kStep, idesc, 1u);                   // hi * lo
                    umma_tf32_ts_pair(d_tmem, a_t + j * UMMA_K, b_d + j * kStep, idesc, 1u);                            // hi * hi
                  }
                  fresh = 0;
                  umma_commit_pair_both(bar_slotfree + 8 * i, 3);
                }
                ++nrun;
              } else {
                // rows [8 kh, 8 kh + 128) of channel block q of the slab: kh image rows = kh * 1024 bytes down
                const uint64_t a_d = a_desc0 + (uint32_t)s * stage16 + (uint32_t)q * slab16 + (uint32_t)kh * (1024 >> 4);
#pragma unroll
                for (int j = 0; j < kSteps; ++j)
                  umma_tf32_pair(d_tmem, a_d + j * kStep, b_d + j * kStep, idesc, (j > 0 || n > 0) ? 1u : 0u);
              }
            }
          }
          if (!ok) break;
          if (!SPLIT3) {
            umma_commit_pair_both(bar_empty + 8 * s, 3);
            if (++s == kStages) { s = 0; ph ^= 1; }
          }
          if (++grp == p.groups) { grp = 0; ++kw; }
        }
        if (!ok) break;
        if (active) {
          umma_commit_pair_both(bar_tfull + 8 * a, 3);
          if (++buf == C::kBufs) { buf = 0; buf_ph ^= 1; }
        }
      }
    }
  } else if (warp >= C::kEpilogueWarp0 && warp < C::kSplitWarp0) {
    // ------------------------------- epilogue (both CTAs, own 128 pixels) -------------------------------
    const int quarter = warp & 3;
    const int col0 = ((warp - C::kEpilogueWarp0) >> 2) * 32;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)col0;
    const uint32_t tempty0 = rank == 0 ? bar_tempty : map_to_cta(bar_tempty, 0);
    const int64_t plane = (int64_t)p.OH * p.OW;
    int buf = 0;
    uint32_t buf_ph = 0;  // TF32: phase of the accumulator pair in use; 3xTF32: bit i = phase of accumulator i
    int64_t nrun = 0;     // 3xTF32: running k-block number of this pair at the start of the tile
    bool ok = true;
    const int chunk = SPLIT3 ? p.chunk_kb : p.num_kb;
    for (int64_t tile = pair; tile < p.num_tiles && ok; tile += num_pairs) {
      float sum[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) sum[j] = 0.f;
      for (int kb0 = 0; kb0 < p.num_kb; kb0 += chunk) {
        // 3xTF32: an accumulator takes part in the chunk if its issuer owned a k-block of it
        const int kb1 = kb0 + chunk < p.num_kb ? kb0 + chunk : p.num_kb;
        bool act[C::kIssuers];
#pragma unroll
        for (int i = 0; i < C::kIssuers; ++i) {
          act[i] = !SPLIT3 || chunk_has(i, nrun + kb0, nrun + kb1);
          const uint32_t ph = SPLIT3 ? (buf_ph >> i) & 1u : buf_ph;
          if (ok && act[i]) ok = mbar_wait(bar_tfull + 8 * (C::kBufs * i + buf), ph, abort_flag, p.status, 8u);
        }
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 32; c += 16) {
          // accumulators are read kLdGroup at a time (register budget: 672 threads in 3xTF32 mode)
          constexpr int kLdGroup = SPLIT3 ? 2 : C::kIssuers;
#pragma unroll
          for (int i0 = 0; i0 < C::kIssuers; i0 += kLdGroup) {
            uint32_t v[kLdGroup][16];
#pragma unroll
            for (int i = 0; i < kLdGroup; ++i)
              tmem_ld16(lane_addr + (uint32_t)((C::kBufs * (i0 + i) + buf) * kAccCols + c), v[i]);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float t = 0.f;
#pragma unroll
              for (int i = 0; i < kLdGroup; ++i) t += act[i0 + i] ? __uint_as_float(v[i][j]) : 0.f;
              sum[c + j] += t;
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
#pragma unroll
          for (int i = 0; i < C::kIssuers; ++i) {
            if (!act[i]) continue;
            if (rank == 0) mbar_arrive(bar_tempty + 8 * (C::kBufs * i + buf));
            else mbar_arrive_cluster_relaxed(tempty0 + 8 * (C::kBufs * i + buf));
          }
        }
        if (SPLIT3) {
#pragma unroll
          for (int i = 0; i < C::kIssuers; ++i)
            if (act[i]) buf_ph ^= 1u << i;
        } else if (++buf == C::kBufs) {
          buf = 0;
          buf_ph ^= 1;
        }
      }
      nrun += p.num_kb;
      if (!ok) break;
      // this thread's output pixel: row r of the tile is pixel (r / 8, r % 8)
      const int64_t ct = 2 * tile + (int64_t)rank;
      const int img = (int)(ct / p.tiles_per_img);
      const int rem = (int)(ct - (int64_t)img * p.tiles_per_img);
      const int ty = rem / p.tiles_w;
      const int oh = ty * TH + (row >> 3), ow = (rem - ty * p.tiles_w) * TW + (row & 7);
      if (ct < p.total_tiles && oh < p.OH && ow < p.OW && col0 < p.M) {
        const int ncols = p.M - col0 < 32 ? p.M - col0 : 32;
        if (p.epilogue != B200_EPI_NONE) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 b = *reinterpret_cast<const float4 *>(&s_bias[col0 + j]);
            sum[j] += b.x; sum[j + 1] += b.y; sum[j + 2] += b.z; sum[j + 3] += b.w;
          }
          if (p.epilogue == B200_EPI_BIAS_RELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) sum[j] = fmaxf(sum[j], 0.f);
          }
        }
        if (p.y_nhwc) {
          float *y = p.Y + (((int64_t)img * p.OH + oh) * p.OW + ow) * p.M + col0;
          if (ncols == 32 && p.vec8) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) st_global_v8(y + j, &sum[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < ncols) y[j] = sum[j];
          }
        } else {
          // NCHW: for a fixed channel the 32 lanes hold 4 rows x 8 consecutive pixels = four whole 32-byte sectors
          float *y = p.Y + ((int64_t)img * p.M + col0) * plane + (int64_t)oh * p.OW + ow;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < ncols) y[j * plane] = sum[j];
        }
      }
      __syncwarp();  // the warp-wide TMEM loads of the next tile need every lane back
    }
  } else if (SPLIT3 && warp >= C::kSplitWarp0) {
    // ------------------------------- split warps: A -> hi / lo halves in TMEM -------------------------------
    // Two groups of four warps (one warp per TMEM lane quarter, one pixel row per thread). Group g converts the
    // k-blocks whose running number has parity g, so two k-blocks are in conversion at any time: one warp's
    // load -> convert -> wait for the slot -> tcgen05.st -> publish chain is longer than the MMAs of a k-block.
    const int quarter = warp & 3;
    const int group = (warp - C::kSplitWarp0) >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t a_lane = tmem_base + ((uint32_t)(quarter * 32) << 16) + C::kSlotCol0;
    const uint32_t split0 = rank == 0 ? bar_split : map_to_cta(bar_split, 0);
    int s = 0;
    uint32_t ph = 0;
    int64_t n = 0;  // running k-block number of this CTA: slot n % kSlots, converted by group n % 2
    bool ok = true;
    for (int64_t tile = pair; tile < p.num_tiles && ok; tile += num_pairs) {
      int grp = 0;
      for (int st = 0; st < p.stages_per_tile && ok; ++st) {
        if (!(ok = mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 16u))) break;
        const int nkb = p.cblocks - grp * 2 < p.kbs ? p.cblocks - grp * 2 : p.kbs;
        for (int q = 0; q < nkb && ok; ++q) {
          for (int kh = 0; kh < p.KH; ++kh, ++n) {
            if ((int)(n & 1) != group) continue;
            const int slot = (int)(n & (kSlots - 1));
            const uint32_t slot_ph = (uint32_t)((n / kSlots) & 1);
            // this thread's pixel under filter row kh: slab row 8 kh + row of channel block q
            const int srow = kh * 8 + row;
            const float4 *arow = reinterpret_cast<const float4 *>(stages + (size_t)s * stage_bytes +
                                                                  (size_t)q * p.slab_bytes + (size_t)srow * 128);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              uint32_t hi[16], lo[16];
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                const float4 x = arow[(half * 4 + c) ^ (srow & 7)];
                const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const uint32_t h = split_hi(xs[e]);
                  hi[4 * c + e] = h;
                  lo[4 * c + e] = split_hi(xs[e] - __uint_as_float(h));
                }
              }
              if (half == 0) {
                // the slot was last read by the MMAs of the k-block kSlots before this one
                if (!(ok = mbar_wait(bar_slotfree + 8 * slot, slot_ph ^ 1, abort_flag, p.status, 32u))) break;
                tc_fence_after();
              }
              tmem_st16(a_lane + (uint32_t)slot * 64 + half * 16, hi);
              tmem_st16(a_lane + (uint32_t)slot * 64 + 32 + half * 16, lo);
            }
            if (!ok) break;
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if (rank == 0) mbar_arrive(bar_split + 8 * slot);
              else mbar_arrive_cluster_relaxed(split0 + 8 * slot);
            }
          }
        }
        if (!ok) break;
        // this warp has read all it needs of the stage: hand it back to its producer
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + 8 * s);
        if (++s == kStages) { s = 0; ph ^= 1; }
        if (++grp == p.groups) grp = 0;
      }
    }
  }

  // Teardown: neither CTA may leave while its partner can still signal its barriers or read its shared
  // memory through the pair's MMAs.
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (s_abort) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
  }
  if (warp == 3) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, C::kTmemCols);
  }
}

// OIHW filter -> [Cout][KH*KW][Cp] with the channel axis zero-padded to Cp (a multiple of 32): the K order
// (tap, channel) in which the implicit GEMM walks the input. With `hi` / `lo` also the two TF32 halves.
__global__ void __launch_bounds__(256)
conv_prepare_filter_kernel(const float *__restrict__ w, float *__restrict__ raw, float *__restrict__ hi,
                           float *__restrict__ lo, int64_t M, int C, int taps, int Cp) {
  const int64_t total = M * taps * Cp;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % Cp);
    const int64_t r = i / Cp;
    const int tap = (int)(r % taps);
    const int64_t m = r / taps;
    const float v = c < C ? w[(m * C + c) * taps + tap] : 0.f;
    raw[i] = v;
    if (hi) {
      const float h = to_tf32_rna(v);
      hi[i] = h;
      lo[i] = to_tf32_rna(v - h);
    }
  }
}

inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

struct PairPlan {
  int bn, stages, b_kb_bytes, num_kb, kbs, groups;
  size_t smem;
};

// Does the resident-filter pair kernel cover this convolution, and with which geometry?
bool pair_plan(const b200_conv_desc &d, PairPlan *out) {
  if (d.M < 1 || d.M > 64) return false;
  // the channel axis is described to TMA as {32 within a block, block}: whole blocks, or a single partial one
  if (d.C > 32 && d.C % 32 != 0) return false;
  const bool split3 = d.math_mode == B200_MATH_FP32X3;
  PairPlan pl;
  pl.bn = (int)((d.M + 15) / 16 * 16);
  const int64_t cblocks = (d.C + 31) / 32;
  const int64_t num_kb = d.KH * d.KW * cblocks;
  pl.kbs = cblocks > 1 ? 2 : 1;
  pl.groups = (int)((cblocks + pl.kbs - 1) / pl.kbs);
  pl.b_kb_bytes = (split3 ? 2 : 1) * (pl.bn / 2) * 128;
  const int64_t b_bytes = num_kb * pl.b_kb_bytes;
  const int64_t slab_rows = TH + d.KH - 1;  // image rows of a slab; 8 pixels = 1024 bytes each
  if (slab_rows > 256) return false;        // TMA box extent
  const int64_t stage_bytes = (int64_t)pl.kbs * slab_rows * 1024;
  const int64_t budget = kMaxDynamicSmem - 1024 /*alignment slack*/ - kBarrierBytes;
  if (b_bytes > budget - 2 * stage_bytes) return false;
  int64_t stages = (budget - b_bytes) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (2 * b_bytes > 1000000) return false;  // one mbarrier transaction count holds both CTAs' filter bytes
  if (d.KW * pl.groups > 0x7fffffffLL) return false;
  pl.stages = (int)stages;
  pl.num_kb = (int)num_kb;
  pl.smem = (size_t)(b_bytes + stages * stage_bytes + 1024 + kBarrierBytes);
  *out = pl;
  return true;
}

template <bool SPLIT3>
int max_pairs_for(size_t smem, int *out) {
  using C = PairCfg<SPLIT3>;
  auto kern = conv_pair_kernel<SPLIT3>;
  static std::mutex mu;
  static int cached[64] = {};
  static size_t cached_smem[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(B200_ECUDA, "conv(pair): bad device");
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0 || cached_smem[dev] != smem) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem) != cudaSuccess)
      return fail(B200_ECUDA, "conv(pair): cannot raise the dynamic shared memory limit");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kNumSMs, 1, 1);
    cfg.blockDim = dim3(C::kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1)
      return fail(B200_ECUDA, "conv(pair): cudaOccupancyMaxActiveClusters failed");
    cached[dev] = n;
    cached_smem[dev] = smem;
  }
  *out = cached[dev];
  return B200_OK;
}

template <bool SPLIT3>
int launch_pair_conv(cudaStream_t st, const PairPlan &pl, const CUtensorMap &mx, const CUtensorMap &mw,
                     const CUtensorMap &mwlo, const ConvPairParams &p) {
  int max_pairs = 0;
  if (int rc = max_pairs_for<SPLIT3>(pl.smem, &max_pairs)) return rc;
  const int64_t pairs = p.num_tiles < max_pairs ? p.num_tiles : max_pairs;
  conv_pair_kernel<SPLIT3><<<(unsigned)(2 * pairs), PairCfg<SPLIT3>::kThreads, pl.smem, st>>>(mx, mw, mwlo, p);
  return check_launch("conv_pair");
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// host side: prepared filters, layout flags, dispatch
// ---------------------------------------------------------------------------------------------
size_t conv2d_filter_bytes(const b200_conv_desc &d) {
  // shapes the tensor cores cannot take keep the OIHW filter as it is (the CUDA-core kernel reads it directly)
  if (!conv2d_tc_supported(d, nullptr)) return align256((size_t)d.M * d.C * d.KH * d.KW * 4);
  const size_t one = align256((size_t)d.M * d.KH * d.KW * ((d.C + 31) / 32 * 32) * 4);
  return d.math_mode == B200_MATH_FP32X3 ? 3 * one : one;
}

int conv2d_prepare_filter(cudaStream_t st, const b200_conv_desc &d, const float *W, void *filter, size_t filter_bytes) {
  const size_t need = conv2d_filter_bytes(d);
  if (!filter || filter_bytes < need)
    return fail(B200_EWORKSPACE, "conv: prepared filter needs %zu bytes, %zu given", need, filter_bytes);
  if (!aligned16(filter)) return fail(B200_EINVAL, "conv: prepared filter must be 16-byte aligned");
  if (!conv2d_tc_supported(d, nullptr)) {
    if (cudaMemcpyAsync(filter, W, (size_t)d.M * d.C * d.KH * d.KW * 4, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
      return fail(B200_ECUDA, "conv: copying the filter failed");
    return B200_OK;
  }
  const int Cp = (int)((d.C + 31) / 32 * 32), taps = (int)(d.KH * d.KW);
  const size_t one = align256((size_t)d.M * taps * Cp * 4);
  float *raw = static_cast<float *>(filter);
  float *hi = nullptr, *lo = nullptr;
  if (d.math_mode == B200_MATH_FP32X3) {
    hi = reinterpret_cast<float *>(static_cast<char *>(filter) + one);
    lo = reinterpret_cast<float *>(static_cast<char *>(filter) + 2 * one);
  }
  const int64_t total = d.M * taps * Cp;
  int64_t g = (total + 255) / 256;
  if (g > kNumSMs * 8) g = kNumSMs * 8;
  conv_prepare_filter_kernel<<<(unsigned)g, 256, 0, st>>>(W, raw, hi, lo, d.M, (int)d.C, taps, Cp);
  return check_launch("conv_prepare_filter");
}

bool conv2d_nhwc_supported(const b200_conv_desc &d) {
  PairPlan pl;
  return conv2d_tc_supported(d, nullptr) && pair_plan(d, &pl);
}

size_t conv2d_run_workspace_bytes(const b200_conv_desc &d, int flags) {
  if (!conv2d_tc_supported(d, nullptr) || (flags & B200_CONV_X_NHWC)) return 0;
  return align256((size_t)d.N * d.H * d.W * d.C * 4);  // the NHWC copy of an NCHW input
}

int conv2d_run(cudaStream_t st, const b200_conv_desc &d, int flags, const float *X, const void *filter,
               const float *bias, float *Y, int64_t OH, int64_t OW, void *workspace, size_t workspace_bytes) {
  const bool x_nhwc = (flags & B200_CONV_X_NHWC) != 0, y_nhwc = (flags & B200_CONV_Y_NHWC) != 0;
  PairPlan pl;
  const bool tc = conv2d_tc_supported(d, x_nhwc ? X : nullptr);
  const bool pair = tc && pair_plan(d, &pl);
  if (!tc && !x_nhwc && !y_nhwc) return conv2d_simt(st, d, X, static_cast<const float *>(filter), bias, Y, OH, OW);
  if ((x_nhwc || y_nhwc) && !pair)
    return fail(B200_EUNSUPPORTED, "conv: NHWC tensors are only taken by the resident-filter kernel "
                                   "(at most 64 output channels, filter half within shared memory)");
  if (!aligned16(filter)) return fail(B200_EINVAL, "conv: prepared filter must be 16-byte aligned");
  const float *xt = X;
  if (!x_nhwc) {
    const size_t need = conv2d_run_workspace_bytes(d, flags);
    if (!workspace || workspace_bytes < need)
      return fail(B200_EWORKSPACE, "conv: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    if (!aligned16(workspace)) return fail(B200_EINVAL, "conv: workspace must be 16-byte aligned");
    // NCHW -> NHWC (per image a [C, H*W] -> [H*W, C] transpose), so that the 32 channels of a k-block are
    // contiguous and filter-tap shifts move only the outer TMA coordinates.
    if (int rc = transpose_2d(st, X, static_cast<float *>(workspace), d.N, d.C, d.H * d.W)) return rc;
    xt = static_cast<const float *>(workspace);
  } else if (!aligned16(X)) {
    return fail(B200_EINVAL, "conv: an NHWC input must be 16-byte aligned");
  }
  const int Cp = (int)((d.C + 31) / 32 * 32), taps = (int)(d.KH * d.KW);
  const size_t one = align256((size_t)d.M * taps * Cp * 4);
  const float *w_raw = static_cast<const float *>(filter);
  if (!pair) return conv2d_tc_gemm(st, d, xt, w_raw, bias, Y, OH, OW);

  const bool split3 = d.math_mode == B200_MATH_FP32X3;
  const float *w_hi = split3 ? reinterpret_cast<const float *>(static_cast<const char *>(filter) + one) : w_raw;
  const float *w_lo = split3 ? reinterpret_cast<const float *>(static_cast<const char *>(filter) + 2 * one) : w_raw;
  CUtensorMap mx, mw, mwlo;
  {
    // NHWC input seen as {32 channels of a block, W, H, channel block, N}; one box = the slab of one filter column
    const uint64_t cblocks = (uint64_t)((d.C + 31) / 32);
    uint64_t dims[5] = {(uint64_t)(d.C < 32 ? d.C : 32), (uint64_t)d.W, (uint64_t)d.H, cblocks, (uint64_t)d.N};
    uint64_t str[4] = {(uint64_t)d.C * 4, (uint64_t)d.W * d.C * 4, 128, (uint64_t)d.H * d.W * d.C * 4};
    uint32_t box[5] = {BK, TW, (uint32_t)(TH + d.KH - 1), (uint32_t)pl.kbs, 1};
    if (int rc = encode_map5(&mx, xt, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  }
  {
    uint64_t dims[4] = {(uint64_t)taps * Cp, (uint64_t)d.M, 1, 1};
    uint64_t str[3] = {(uint64_t)taps * Cp * 4, (uint64_t)taps * Cp * 4 * d.M, (uint64_t)taps * Cp * 4 * d.M};
    if (int rc = encode_map(&mw, w_hi, dims, str, BK, (uint32_t)(pl.bn / 2), CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
    if (int rc = encode_map(&mwlo, w_lo, dims, str, BK, (uint32_t)(pl.bn / 2), CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  }
  ConvPairParams p{};
  p.KH = (int)d.KH;
  p.KW = (int)d.KW;
  p.pad_h = (int)d.pad_h;
  p.pad_w = (int)d.pad_w;
  p.OH = (int)OH;
  p.OW = (int)OW;
  p.slab_bytes = (int)((TH + d.KH - 1) * 1024);
  p.tiles_w = (int)((OW + TW - 1) / TW);
  p.tiles_per_img = p.tiles_w * (int)((OH + TH - 1) / TH);
  p.cblocks = Cp / 32;
  p.num_kb = pl.num_kb;
  {
    const int nchunks = (pl.num_kb + kMaxChunkKb - 1) / kMaxChunkKb;
    p.chunk_kb = (pl.num_kb + nchunks - 1) / nchunks;
  }
  p.kbs = pl.kbs;
  p.groups = pl.groups;
  p.stages_per_tile = (int)d.KW * pl.groups;
  p.total_tiles = d.N * p.tiles_per_img;
  p.num_tiles = (p.total_tiles + 1) / 2;
  p.bn = pl.bn;
  p.M = (int)d.M;
  p.stages = pl.stages;
  p.b_kb_bytes = pl.b_kb_bytes;
  p.y_nhwc = y_nhwc ? 1 : 0;
  p.epilogue = d.epilogue;
  p.vec8 = (d.M % 8 == 0 && (reinterpret_cast<uintptr_t>(Y) & 31u) == 0) ? 1 : 0;
  p.bias = bias;
  p.Y = Y;
  p.status = device_status_ptr();
  if (!p.status) return fail(B200_ECUDA, "conv(pair): device status word unavailable");
  if (p.total_tiles > 0x7fffffff00LL) return fail(B200_EUNSUPPORTED, "conv: too many output tiles");
  return split3 ? launch_pair_conv<true>(st, pl, mx, mw, mwlo, p) : launch_pair_conv<false>(st, pl, mx, mw, mwlo, p);
}

}  // namespace b200
