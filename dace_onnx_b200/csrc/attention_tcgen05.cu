// Fused attention for sm_100a: softmax(Q K^T * scale) V per (batch, head) without materialising
// the [S, S] score matrix in HBM. Replaces the node pattern MatMul -> Mul(const) -> Softmax -> MatMul of the
// exported BERT graph (TF32 tensor-core mode).
//
// One persistent CTA per SM walks query tiles of 128 rows, two at a time; Q, K and V arrive by TMA
// (cp.async.bulk.tensor; K as the K-major B operand of Q K^T, V as the MN-major B operand of P V), the scores are
// accumulated in TMEM by tcgen05.mma kind::tf32, the softmax warps turn them into P in place (tcgen05.ld / st),
// and P V reads its A operand from TMEM. HBM traffic is Q, K, V once per query tile (K and V of a head come from
// L2 the second and third time) and the context once: 16 B per (token, head-dim element) instead of the
// 4 * S * S * 4 B per head the unfused chain moves.
//
// All waits are bounded (see tc_common.cuh); on expiry the CTA records the fact in the device
// status word, every role leaves, TMEM is freed and the kernel returns.
#include "common.cuh"
#include "contract.cuh"
#include "tc_common.cuh"


namespace b200 {
using namespace tc;
namespace {

constexpr int kD = 64;                  // head dimension
constexpr int kBlkBytes = 128 * kD * 4; // 32 KiB: 128 rows x 64 fp32 as two slices of [128 rows][128 B]

// ---------------------------------------------------------------------------------------------
// Two query tiles in flight. Per query tile and key block the chain  Q K^T -> softmax -> P V  is serial (P
// overwrites the scores in TMEM, and the next block's scores go to the same columns), and each link is bound by
// latency rather than throughput: one thread issues a tcgen05.mma every ~55-100 clk and pays ~200 clk for every
// barrier wait in between (measured), so the 8 score MMAs and the 2 x 8 P V MMAs of a block take ~800-1000 clk each,
// and the exponentials of a block take the SM's special-function units ~1000 clk (16 per clk). A CTA therefore works
// on two query tiles ("slots") at once, each with its own shared-memory buffers (Q, one key block, one value
// block), its own half of TMEM (scores / P: 128 columns, two partial outputs: 64 + 64) and its own warps:
//   warps 0-1    TMA producer of slot 0 / 1
//   warps 2-3    score issuer of slot 0 / 1:  S = Q K_j^T                          (kind::tf32, A and B in smem)
//   warps 4-7    P V issuers, two per slot: first / second 64 keys of the block into partial output 0 / 1
//                (A = P from TMEM); each starts as soon as its 64 columns of P are published
//   warps 8-15   softmax, four per slot: one score row per thread
//   warps 16-19  output, both slots in turn: add the two partial outputs, divide by the row sum, store (kept off the
//                softmax warps, whose next tile would otherwise wait ~3K clk for the last P V and the stores)
// so that one slot's MMAs run while the other slot's softmax warps are busy. Keys are walked in blocks of 128
// with a running maximum; the exponent offset follows it only when it has grown by more than 2^8, so the
// outputs accumulate in TMEM across blocks and are rescaled rarely. Any sequence length that is a multiple of 32.
// Barriers of a slot (all single-buffered, phase = block or tile count modulo 2):
//   q_full / q_empty, k_full / k_empty, v_full      loads (a value block is free again at pv_done)
//   s_full    score issuer -> softmax          p_full[2]   softmax (one arrival per warp) -> P V issuer 0 / 1
//   pv_done   both P V issuers -> score issuer (score columns free), producer, softmax, output warps
//   l_ready   softmax (row sums of the finished tile in shared memory) -> output warps
//   o_free    output warps (partial outputs read) -> P V issuers (the next tile may overwrite them)
// ---------------------------------------------------------------------------------------------
constexpr int kThreads = 32 * 20;
enum SlotBar { kQFull = 0, kQEmpty, kKFull, kKEmpty, kVFull, kSFull, kPFull0, kPFull1, kPvDone, kLReady, kOFree, kSlotBars };

struct AttnParams {
  int S, heads, n_blocks;
  int64_t tiles;  // batch * heads * n_blocks query tiles
  float scale_log2e;
  float *out;
  int64_t o_batch, o_row, o_head;
  unsigned *status;
};

// exp2 of 32 scores (scaled, offset subtracted) in place; four partial sums break the dependency chain of the row sum
__device__ __forceinline__ void exp32_inplace(uint32_t (&v)[32], float c, float off, float (&sum)[4]) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(fmaf(__uint_as_float(v[i]), c, -off)));
    sum[i & 3] += e;
    v[i] = __float_as_uint(e);
  }
}

__global__ void __launch_bounds__(kThreads, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t smem0 = smem_u32(smem);  // Q0 Q1 K0 K1 V0 V1, 32 KiB each
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + 6 * (size_t)kBlkBytes);
  const uint32_t bar0 = smem_u32(bars);
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ float s_rowsum[2][128];  // [slot][row]: row sums of the tile the output warps are about to finish
  __shared__ int s_exp_turn[4];  // per scheduler: which slot's softmax warp is in its exponential pass (0 = none)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < 4; ++i) s_exp_turn[i] = 0;
    for (int s = 0; s < 2; ++s)
      for (int i = 0; i < kSlotBars; ++i)
        mbar_init(bar0 + 8 * (s * kSlotBars + i),
                  (i == kPFull0 || i == kPFull1 || i == kLReady || i == kOFree) ? 4 : (i == kPvDone ? 2 : 1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&s_tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int *abort_flag = &s_abort;
  const int nb = p.n_blocks;
  // role and slot of this warp
  const int slot = warp < 2 ? warp : (warp < 4 ? warp - 2 : (warp < 8 ? (warp - 4) >> 1 : (warp < 16 ? (warp - 8) >> 2 : 0)));
  const uint32_t bar = bar0 + 8 * (slot * kSlotBars);
  const uint32_t q_smem = smem0 + slot * kBlkBytes, k_smem = smem0 + (2 + slot) * kBlkBytes,
                 v_smem = smem0 + (4 + slot) * kBlkBytes;
  const uint32_t s_tmem = tmem_base + slot * 256, o0_tmem = s_tmem + 128, o1_tmem = s_tmem + 192;
  const int64_t t0 = 2 * (int64_t)blockIdx.x + slot, t_step = 2 * (int64_t)gridDim.x;
  bool ok = true;

  if (warp < 2) {
    // ------------------------------- TMA producer of the slot -------------------------------
    if (lane == 0) {
      int64_t n = 0, g = 0;
      for (int64_t t = t0; t < p.tiles && ok; t += t_step, ++n) {
        const int64_t item = t / nb;
        const int mt = (int)(t - item * nb), b = (int)(item / p.heads), h = (int)(item % p.heads);
        if (!(ok = mbar_wait(bar + 8 * kQEmpty, (uint32_t)(n & 1) ^ 1, abort_flag, p.status, 1u))) break;
        mbar_expect_tx(bar + 8 * kQFull, kBlkBytes);
        tma_load_4d(q_smem, &map_q, bar + 8 * kQFull, 0, mt * 128, h, b);
        tma_load_4d(q_smem + kBlkBytes / 2, &map_q, bar + 8 * kQFull, 32, mt * 128, h, b);
        for (int j = 0; j < nb; ++j, ++g) {
          const uint32_t ph = (uint32_t)(g & 1);
          if (!(ok = mbar_wait(bar + 8 * kKEmpty, ph ^ 1, abort_flag, p.status, 1u))) break;
          mbar_expect_tx(bar + 8 * kKFull, kBlkBytes);
          tma_load_4d(k_smem, &map_k, bar + 8 * kKFull, 0, j * 128, h, b);
          tma_load_4d(k_smem + kBlkBytes / 2, &map_k, bar + 8 * kKFull, 32, j * 128, h, b);
          if (!(ok = mbar_wait(bar + 8 * kPvDone, ph ^ 1, abort_flag, p.status, 1u))) break;  // value buffer free
          mbar_expect_tx(bar + 8 * kVFull, kBlkBytes);
          tma_load_4d(v_smem, &map_v, bar + 8 * kVFull, 0, j * 128, h, b);
          tma_load_4d(v_smem + kBlkBytes / 2, &map_v, bar + 8 * kVFull, 32, j * 128, h, b);
        }
      }
    }
  } else if (warp < 4) {
    // ------------------------------- score issuer of the slot -------------------------------
    if (lane == 0) {
      const uint32_t idesc_full = make_idesc(128, false);
      const uint64_t kdesc0 = make_smem_desc(0, 16, 1024, kLayoutSw128);
      const uint64_t a_base = kdesc0 + (q_smem >> 4), b_base = kdesc0 + (k_smem >> 4);
      int64_t n = 0, g = 0;
      for (int64_t t = t0; t < p.tiles && ok; t += t_step, ++n) {
        if (!(ok = mbar_wait(bar + 8 * kQFull, (uint32_t)(n & 1), abort_flag, p.status, 2u))) break;
        for (int j = 0; j < nb; ++j, ++g) {
          const uint32_t ph = (uint32_t)(g & 1);
          if (!(ok = mbar_wait(bar + 8 * kKFull, ph, abort_flag, p.status, 2u))) break;
          // the score columns still hold the previous block's P until its P V products are done
          if (!(ok = mbar_wait(bar + 8 * kPvDone, ph ^ 1, abort_flag, p.status, 2u))) break;
          tc_fence_after();
          const int n_len = p.S - j * 128;
          const uint32_t idesc_s = n_len >= 128 ? idesc_full : make_idesc(n_len, false);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            constexpr uint32_t kHalf = (kBlkBytes / 2) >> 4;
            const uint32_t off = (ks >> 2) * kHalf + (ks & 3) * 2;
            umma_tf32(s_tmem, a_base + off, b_base + off, idesc_s, ks > 0 ? 1u : 0u);
          }
          umma_commit(bar + 8 * kSFull);
          umma_commit(bar + 8 * kKEmpty);
          if (j == nb - 1) umma_commit(bar + 8 * kQEmpty);
        }
      }
    }
  } else if (warp < 8) {
    // ------------------------------- P V issuers of the slot -------------------------------
    if (lane == 0) {
      const int second = (warp - 4) & 1;
      const uint32_t o_tmem = second ? o1_tmem : o0_tmem;
      const uint32_t idesc_o = make_idesc(kD, true);
      const uint64_t v_base = make_smem_desc(0, kBlkBytes / 2, 512, kLayoutSw128Base32) + (v_smem >> 4);
      const uint32_t p_bar = bar + 8 * (second ? kPFull1 : kPFull0);
      int64_t g = 0, n = 0;
      for (int64_t t = t0; t < p.tiles && ok; t += t_step, ++n) {
        uint32_t started = 0;  // 0 until this accumulator has received its first product of the tile
        for (int j = 0; j < nb; ++j, ++g) {
          const uint32_t ph = (uint32_t)(g & 1);
          if (!(ok = mbar_wait(bar + 8 * kVFull, ph, abort_flag, p.status, 4u))) break;
          if (!(ok = mbar_wait(p_bar, ph, abort_flag, p.status, 4u))) break;
          // the previous tile's partial outputs must have been read before the first product overwrites them
          if (j == 0 && !(ok = mbar_wait(bar + 8 * kOFree, (uint32_t)(n & 1) ^ 1, abort_flag, p.status, 4u))) break;
          tc_fence_after();
          const int k_len = p.S - j * 128 < 128 ? p.S - j * 128 : 128;
          // 8 key rows of V (8 x 128 B = 64 descriptor units) and 8 columns of P per MMA
          const int k8_lo = second ? 8 : 0, k8_hi = second ? k_len / 8 : (k_len / 8 < 8 ? k_len / 8 : 8);
          if (k8_hi - k8_lo == 8) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const int k8 = k8_lo + q;
              umma_tf32_ts(o_tmem, s_tmem + k8 * 8, v_base + k8 * 64, idesc_o, q > 0 ? 1u : started);
            }
            started = 1;
          } else {
            for (int k8 = k8_lo; k8 < k8_hi; ++k8) {
              umma_tf32_ts(o_tmem, s_tmem + k8 * 8, v_base + k8 * 64, idesc_o, started);
              started = 1;
            }
          }
          umma_commit(bar + 8 * kPvDone);
        }
      }
    }
  } else if (warp < 16) {
    // ------------------------------- softmax of the slot -------------------------------
    // One score row per thread (warp w of the slot's four reads TMEM lanes 32 w ...): no exchange between threads.
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_addr = s_tmem + lane_off;
    const float c = p.scale_log2e;
    int64_t g = 0;
    for (int64_t t = t0; t < p.tiles && ok; t += t_step) {
      float m_run = -INFINITY, l_run = 0.f;
      for (int j = 0; j < nb; ++j, ++g) {
        const uint32_t ph = (uint32_t)(g & 1);
        const int k_len = p.S - j * 128 < 128 ? p.S - j * 128 : 128;  // a multiple of 32
        if (!(ok = mbar_wait(bar + 8 * kSFull, ph, abort_flag, p.status, 8u))) break;
        tc_fence_after();
        // ---- row maximum of the block: two 32-column chunks per TMEM round trip, four partial maxima ----
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (k_len == 128) {
#pragma unroll 1
          for (int c0 = 0; c0 < 128; c0 += 64) {
            uint32_t v0[32], v1[32];
            tmem_ld32(s_addr + c0, v0);
            tmem_ld32(s_addr + c0 + 32, v1);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i)
              mx[i & 3] = fmaxf(mx[i & 3], fmaxf(__uint_as_float(v0[i]), __uint_as_float(v1[i])));
          }
        } else {
#pragma unroll 1
          for (int c0 = 0; c0 < k_len; c0 += 32) {
            uint32_t v0[32];
            tmem_ld32(s_addr + c0, v0);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(v0[i]));
          }
        }
        const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        // lazy exponent offset: follows the running maximum only when that has grown by more than 2^8
        const bool grow = j == 0 || (m_blk - m_run) * c > 8.0f;
        const float m_new = grow ? m_blk : m_run;
        float alpha = 1.0f;
        if (grow) asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(alpha) : "f"((m_run - m_new) * c));
        if (j == 0) alpha = 0.f;
        const float off = m_new * c;
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          // the outputs hold the earlier blocks' sums relative to the old offset; their last P V is long done (this
          // block's scores were issued after it), the wait orders this thread's TMEM accesses after it
          if (!(ok = mbar_wait(bar + 8 * kPvDone, ph ^ 1, abort_flag, p.status, 8u))) break;
          tc_fence_after();
#pragma unroll 1
          for (int q = 0; q < 4; ++q) {
            uint32_t o[32];
            const uint32_t o_addr = o0_tmem + lane_off + q * 32;  // the two partial outputs are adjacent: 128 columns
            tmem_ld32(o_addr, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(o_addr, o);
          }
        }
        // ---- P = exp2(s * c - off) in place, 64 columns (one P V issuer's share) at a time ----
        // The two slots' warps of one scheduler share its special-function unit; taking turns keeps the slots in
        // anti-phase (one in its exponentials while the other's MMAs run) instead of both at half speed.
        if (lane == 0) {
          const long long t_lock = clock64();
          while (atomicCAS(&s_exp_turn[quarter], 0, 1) != 0) {
            if (*abort_flag) break;
            if (clock64() - t_lock > kWaitCycleBudget) {
              *abort_flag = 1;
              atomicOr(p.status, 8u);
              break;
            }
          }
        }
        __syncwarp();
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
        for (int hb = 0; hb < 2; ++hb) {
          if (k_len == 128) {
            uint32_t v0[32], v1[32];
            tmem_ld32(s_addr + hb * 64, v0);
            tmem_ld32(s_addr + hb * 64 + 32, v1);
            tmem_ld_wait();
            exp32_inplace(v0, c, off, sum);
            tmem_st32(s_addr + hb * 64, v0);
            exp32_inplace(v1, c, off, sum);
            tmem_st32(s_addr + hb * 64 + 32, v1);
            tmem_st_wait();
          } else {
            const int c_end = hb * 64 + 64 < k_len ? hb * 64 + 64 : k_len;
#pragma unroll 1
            for (int c0 = hb * 64; c0 < c_end; c0 += 32) {
              uint32_t v0[32];
              tmem_ld32(s_addr + c0, v0);
              tmem_ld_wait();
              exp32_inplace(v0, c, off, sum);
              tmem_st32(s_addr + c0, v0);
            }
            tmem_st_wait();
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar + 8 * (hb ? kPFull1 : kPFull0));
        }
        if (lane == 0) atomicExch(&s_exp_turn[quarter], 0);
        l_run = l_run * alpha + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
        m_run = m_new;
      }
      if (!ok) break;
      // hand the tile's row sums to the output warps (they waited for o_free's predecessor, so the previous tile's
      // sums have been read) and go on with the next tile
      s_rowsum[slot][row_in_tile] = l_run;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar + 8 * kLReady);
    }
  } else {
    // ------------------------------- output, both slots in turn -------------------------------
    // Tile i of slot 0, tile i of slot 1, tile i + 1 of slot 0, ...: once the tile's last P V is complete, add the
    // two partial outputs, release them (o_free), divide by the row sum and store [row, head * 64 ... + 64).
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    for (int64_t i = 0; ok; ++i) {
      const int64_t ta = 2 * (int64_t)blockIdx.x + i * t_step;
      if (ta >= p.tiles) break;  // slot 0 has no tile i: slot 1 has none either
#pragma unroll 1
      for (int sl = 0; sl < 2 && ok; ++sl) {
        const int64_t t = ta + sl;
        if (t >= p.tiles) break;
        const uint32_t sbar = bar0 + 8 * (sl * kSlotBars);
        const uint32_t o_tmem = tmem_base + sl * 256 + 128 + lane_off;  // partial outputs: columns [128, 192), [192, 256)
        if (!(ok = mbar_wait(sbar + 8 * kLReady, (uint32_t)(i & 1), abort_flag, p.status, 16u))) break;
        if (!(ok = mbar_wait(sbar + 8 * kPvDone, (uint32_t)(((i + 1) * nb - 1) & 1), abort_flag, p.status, 16u))) break;
        tc_fence_after();
        const float inv = 1.0f / s_rowsum[sl][row_in_tile];
        const int64_t item = t / nb;
        const int mt = (int)(t - item * nb), b = (int)(item / p.heads), h = (int)(item % p.heads);
        const int row = mt * 128 + row_in_tile;
        float *orow = p.out + (int64_t)b * p.o_batch + (int64_t)row * p.o_row + (int64_t)h * p.o_head;
#pragma unroll 1
        for (int c0 = 0; c0 < kD; c0 += 32) {  // 32 output columns at a time (register budget)
          uint32_t o[32];
          tmem_ld32(o_tmem + c0, o);
          if (p.S > 64) {  // the second partial output exists once a block has more than 64 keys
            uint32_t o2[32];
            tmem_ld32(o_tmem + 64 + c0, o2);
            tmem_ld_wait();
#pragma unroll
            for (int k = 0; k < 32; ++k) o[k] = __float_as_uint(__uint_as_float(o[k]) + __uint_as_float(o2[k]));
          }
          tmem_ld_wait();
          if (c0 + 32 >= kD) {  // everything read: the next tile's P V may overwrite the partial outputs
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(sbar + 8 * kOFree);
          }
          if (row < p.S) {
#pragma unroll
            for (int k = 0; k < 32; k += 8) {
              float r[8];
#pragma unroll
              for (int q = 0; q < 8; ++q) r[q] = __uint_as_float(o[k + q]) * inv;
              asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(orow + c0 + k), "f"(r[0]), "f"(r[1]),
                           "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]), "f"(r[7])
                           : "memory");
            }
          }
        }
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (s_abort) {
    const long long t_abort = clock64();
    while (clock64() - t_abort < 2000000LL) __nanosleep(1000);
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

int encode_qkv_map(CUtensorMap *map, const float *base, const b200_attention_desc &d, int64_t row, int64_t head,
                   int64_t batch, CUtensorMapSwizzle swizzle) {
  uint64_t dims[4] = {(uint64_t)d.head_dim, (uint64_t)d.seq, (uint64_t)d.heads, (uint64_t)d.batch};
  uint64_t str[3] = {(uint64_t)row * 4, (uint64_t)head * 4, (uint64_t)batch * 4};
  // extent-1 axes may carry a zero stride from the caller; give them a harmless valid one
  const uint64_t fb = (uint64_t)row * 4 * (uint64_t)d.seq;
  if (d.heads == 1 && str[1] == 0) str[1] = fb;
  if (d.batch == 1 && str[2] == 0) str[2] = fb;
  return encode_map(map, base, dims, str, 32, 128, swizzle);
}

}  // namespace

bool attention_tc_supported(const b200_attention_desc &d, const float *Q, const float *K, const float *V,
                            const float *out) {
  auto ok4 = [](int64_t v) { return v % 4 == 0; };
  auto ok8 = [](int64_t v) { return v % 8 == 0; };
  if (d.math_mode != B200_MATH_TF32) return false;
  if (d.head_dim != kD || d.seq < 32 || d.seq > 0x7fffff00LL || d.seq % 32 != 0) return false;
  if (d.batch < 1 || d.heads < 1 || d.batch > 0x7fffffffLL || d.heads > 0x7fffffffLL) return false;
  if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || (reinterpret_cast<uintptr_t>(out) & 31u)) return false;
  if (!ok4(d.q_row) || !ok4(d.q_head) || !ok4(d.q_batch) || !ok4(d.k_row) || !ok4(d.k_head) || !ok4(d.k_batch) ||
      !ok4(d.v_row) || !ok4(d.v_head) || !ok4(d.v_batch))
    return false;
  if (!ok8(d.o_row) || !ok8(d.o_head) || !ok8(d.o_batch)) return false;
  if (d.q_row < kD || d.k_row < kD || d.v_row < kD || d.o_row < kD) return false;
  return true;
}

int attention_tc(cudaStream_t st, const b200_attention_desc &d, const float *Q, const float *K, const float *V,
                 float *out) {
  CUtensorMap mq, mk, mv;
  if (int rc = encode_qkv_map(&mq, Q, d, d.q_row, d.q_head, d.q_batch, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = encode_qkv_map(&mk, K, d, d.k_row, d.k_head, d.k_batch, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = encode_qkv_map(&mv, V, d, d.v_row, d.v_head, d.v_batch, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) return rc;
  AttnParams p{};
  p.S = (int)d.seq;
  p.heads = (int)d.heads;
  p.n_blocks = (int)((d.seq + 127) / 128);
  p.tiles = d.batch * d.heads * p.n_blocks;
  p.scale_log2e = d.scale * 1.4426950408889634f;
  p.out = out;
  p.o_batch = d.o_batch;
  p.o_row = d.o_row;
  p.o_head = d.o_head;
  p.status = device_status_ptr();
  if (!p.status) return fail(B200_ECUDA, "attention: device status word unavailable");
  const int smem = 6 * kBlkBytes + 1024 + 256;
  if (cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return fail(B200_ECUDA, "attention: cannot set dynamic shared memory to %d", smem);
  const int64_t ctas = (p.tiles + 1) / 2;  // two query tiles in flight per CTA
  attention_tc_kernel<<<(unsigned)(ctas < kNumSMs ? ctas : kNumSMs), kThreads, smem, st>>>(mq, mk, mv, p);
  return check_launch("attention_tc");
}

}  // namespace b200
