// Fused attention for sm_100a: softmax(Q K^T * scale) V per (batch, head) without materialising
// the [S, S] score matrix in HBM. Replaces the node pattern MatMul -> Mul(const) -> Softmax -> MatMul of the
// exported BERT graph (TF32 tensor-core mode). Two kernels: attention_tc_kernel, described here, keeps a query
// tile's whole score rows in TMEM (S <= 384); attention_stream_kernel (further down) walks the keys in blocks
// with a running maximum (any S).
//
// One persistent CTA per SM walks (batch, head) items, 128 query rows at a time. Q is double
// buffered; the head's K and V stream through a ring of 128-row blocks (K as the K-major B operand
// of Q K^T, V as the MN-major B operand of P V), so loads run ahead of the MMAs across tiles and
// heads. Per query tile:
//   warp 0 loads Q, the key blocks and the value blocks                      (cp.async.bulk.tensor)
//   warps 1 and 10 issue Q K^T block by block into TMEM columns [0, S)  (tcgen05.mma kind::tf32, A and B in
//             smem): warp 1 the even key blocks, warp 10 the odd ones
//   warps 2-9 (two per score row, alternating 32-column blocks) read the row from TMEM, take its
//             maximum, overwrite it in place with P = exp2((s - max) * scale * log2 e) and sum P
//             (tcgen05.ld / st)
//   warps 1 and 10 issue P V with the A operand read from TMEM, 128 key columns at a time as soon as the softmax
//             warps have published them: warp 1 the first 64 keys of a group into columns [384, 448), warp 10
//             the rest into [448, 512). (One thread issues an MMA every ~100 clk, and the 48 N = 64 products of a
//             tile were the longest phase; two threads on two accumulators halve it.)
//   warps 2-9 add the two partial outputs, divide by the row sum and store [row, head*64 .. +64).
// HBM traffic is Q, K, V once and the context once: 16 B per (token, head-dim element) instead of
// the 4 * S * S * 4 B per head the unfused chain moves.
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
constexpr int kRing = 5;                // K / V blocks in flight (shared memory: (2 + kRing) x 32 KiB)
constexpr int kOCol = 384;              // TMEM columns of the two partial output accumulators: [384, 448), [448, 512)
constexpr int kOCol2 = 448;
constexpr int kMaxS = 384;
constexpr int kThreads = 32 * (2 + 8 + 1);   // producer, MMA issuer, 8 softmax / output warps, second MMA issuer

struct AttnParams {
  int S;              // sequence length
  int heads;
  int n_blocks;       // ceil(S / 128): query tiles per head, and key / value blocks per tile
  int64_t items;      // batch * heads
  float scale_log2e;
  float *out;
  int64_t o_batch, o_row, o_head;  // element strides of the output
  unsigned *status;
};

__global__ void __launch_bounds__(kThreads, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t q_smem = smem_u32(smem);                   // two query-tile buffers
  const uint32_t ring_smem = q_smem + 2 * kBlkBytes;        // kRing blocks of K or V
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (2 + kRing) * (size_t)kBlkBytes);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_q_full = bar0, bar_q_empty = bar0 + 16, bar_ring_full = bar0 + 32,
                 bar_ring_empty = bar_ring_full + 8 * kRing, bar_s_full = bar_ring_empty + 8 * kRing,
                 bar_o_full = bar_s_full + 8, bar_o_empty = bar_s_full + 16, bar_p_full = bar_s_full + 24;  // [4]
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ float s_red[2][128];  // row maximum / row sum exchange between the two warps of a lane quarter
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    s_abort = 0;
    // barriers the two issuing threads signal together take two arrivals
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_q_full + 8 * i, 1);
      mbar_init(bar_q_empty + 8 * i, 2);
    }
    for (int i = 0; i < kRing; ++i) {
      mbar_init(bar_ring_full + 8 * i, 1);
      mbar_init(bar_ring_empty + 8 * i, 2);
    }
    mbar_init(bar_s_full, 2);
    mbar_init(bar_o_full, 2);
    mbar_init(bar_o_empty, 256);
    for (int c = 0; c < 4; ++c) mbar_init(bar_p_full + 8 * c, 256);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&s_tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int *abort_flag = &s_abort;
  const int n_chunks = p.n_blocks;  // 128-column groups of P, one per value block

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    // Per query tile: Q (32 KiB), then the key blocks, then the value blocks of the head, each
    // 128 rows x 64 as two [128][128 B] slices. K and V are re-read for every query tile of the
    // head (they come from L2 the second and third time); in exchange every load runs ahead of
    // the MMAs through the ring, across tiles and heads.
    if (lane == 0) {
      int rs = 0, qs = 0;
      uint32_t r_ph = 0, q_ph = 0;
      bool ok = true;
      for (int64_t item = blockIdx.x; item < p.items && ok; item += gridDim.x) {
        const int b = (int)(item / p.heads), h = (int)(item % p.heads);
        for (int mt = 0; mt < p.n_blocks && ok; ++mt) {
          if (!(ok = mbar_wait(bar_q_empty + 8 * qs, q_ph ^ 1, abort_flag, p.status, 1u))) break;
          mbar_expect_tx(bar_q_full + 8 * qs, kBlkBytes);
          tma_load_4d(q_smem + qs * kBlkBytes, &map_q, bar_q_full + 8 * qs, 0, mt * 128, h, b);
          tma_load_4d(q_smem + qs * kBlkBytes + kBlkBytes / 2, &map_q, bar_q_full + 8 * qs, 32, mt * 128, h, b);
          if (++qs == 2) { qs = 0; q_ph ^= 1; }
          for (int j = 0; j < 2 * p.n_blocks; ++j) {
            const bool is_v = j >= p.n_blocks;
            const int r0 = (is_v ? j - p.n_blocks : j) * 128;
            if (!(ok = mbar_wait(bar_ring_empty + 8 * rs, r_ph ^ 1, abort_flag, p.status, 1u))) break;
            mbar_expect_tx(bar_ring_full + 8 * rs, kBlkBytes);
            const uint32_t dst = ring_smem + rs * kBlkBytes;
            const CUtensorMap *map = is_v ? &map_v : &map_k;
            tma_load_4d(dst, map, bar_ring_full + 8 * rs, 0, r0, h, b);
            tma_load_4d(dst + kBlkBytes / 2, map, bar_ring_full + 8 * rs, 32, r0, h, b);
            if (++rs == kRing) { rs = 0; r_ph ^= 1; }
          }
        }
      }
    }
  } else if (warp == 1 || warp == 10) {
    // ------------------------------- MMA issuers -------------------------------
    // Both threads walk the same sequence of ring slots; `second` decides which score blocks and which half of
    // every P V group are this thread's. A key block is released by its one consumer with two commits, a value
    // block by one commit of each thread (every ring barrier takes two arrivals).
    if (lane == 0) {
      const int second = warp == 10 ? 1 : 0;
      int rs = 0, qs = 0;
      uint32_t r_ph = 0, q_ph = 0, t_ph = 0;  // t_ph: phase of the per-tile barriers (o_empty, p_full, o_full)
      // Descriptors are built once; inside the loops an MMA costs one 64-bit add on its operand
      // descriptors (the start-address field counts 16-byte units), because the issuing thread's
      // instruction latency, not the tensor core, would otherwise bound the small MMAs.
      const uint32_t idesc_o = make_idesc(kD, true);
      const uint32_t idesc_full = make_idesc(128, false);
      const uint64_t kdesc0 = make_smem_desc(0, 16, 1024, kLayoutSw128);                    // Q and K blocks
      const uint64_t vdesc0 = make_smem_desc(0, kBlkBytes / 2, 512, kLayoutSw128Base32);   // V blocks
      const uint32_t o_tmem = tmem_base + (second ? kOCol2 : kOCol);
      bool ok = true;
      for (int64_t item = blockIdx.x; item < p.items && ok; item += gridDim.x) {
        for (int mt = 0; mt < p.n_blocks && ok; ++mt) {
          if (!(ok = mbar_wait(bar_q_full + 8 * qs, q_ph, abort_flag, p.status, 2u))) break;
          const uint64_t a_base = kdesc0 + ((q_smem + qs * kBlkBytes) >> 4);
          // S[:, 128 j .. ] = Q K_j^T, one key block at a time as it lands; block j belongs to thread j % 2
          for (int j = 0; j < p.n_blocks && ok; ++j) {
            if ((j & 1) == second) {
              if (!(ok = mbar_wait(bar_ring_full + 8 * rs, r_ph, abort_flag, p.status, 2u))) break;
              tc_fence_after();
              const int n_len = p.S - j * 128;
              const uint32_t idesc_s = n_len >= 128 ? idesc_full : make_idesc(n_len, false);
              const uint64_t b_base = kdesc0 + ((ring_smem + rs * kBlkBytes) >> 4);
              const uint32_t d_tmem = tmem_base + j * 128;
#pragma unroll
              for (int ks = 0; ks < 8; ++ks) {
                // k-block kb = ks / 4 is half a block further (kBlkBytes / 2), k-step kk = ks % 4 is 32 B further
                constexpr uint32_t kHalf = (kBlkBytes / 2) >> 4;
                const uint32_t off = (ks >> 2) * kHalf + (ks & 3) * 2;
                umma_tf32(d_tmem, a_base + off, b_base + off, idesc_s, ks > 0 ? 1u : 0u);
              }
              umma_commit(bar_ring_empty + 8 * rs);
              umma_commit(bar_ring_empty + 8 * rs);
            }
            if (++rs == kRing) { rs = 0; r_ph ^= 1; }
          }
          if (!ok) break;
          umma_commit(bar_q_empty + 8 * qs);  // Q buffer reusable once both threads' products have read it
          umma_commit(bar_s_full);            // scores ready for the softmax warps (both threads' blocks)
          if (++qs == 2) { qs = 0; q_ph ^= 1; }
          // O = P V, A operand (P) from TMEM; the previous tile's O must have been read out
          if (!(ok = mbar_wait(bar_o_empty, t_ph ^ 1, abort_flag, p.status, 2u))) break;
          uint32_t started = 0;  // 0 until this thread's accumulator has received its first product of the tile
          for (int c = 0; c < n_chunks && ok; ++c) {
            if (!(ok = mbar_wait(bar_p_full + 8 * c, t_ph, abort_flag, p.status, 4u))) break;
            if (!(ok = mbar_wait(bar_ring_full + 8 * rs, r_ph, abort_flag, p.status, 4u))) break;
            tc_fence_after();
            const uint64_t v_base = vdesc0 + ((ring_smem + rs * kBlkBytes) >> 4);
            const uint32_t p_tmem = tmem_base + c * 128;
            const int k_len = p.S - c * 128 < 128 ? p.S - c * 128 : 128;
            // 8 key rows of V (8 x 128 B = 64 descriptor units) and 8 columns of P per MMA; this thread's keys
            // are [0, 64) or [64, 128) of the group
            const int k8_lo = second ? 8 : 0, k8_hi = second ? k_len / 8 : (k_len / 8 < 8 ? k_len / 8 : 8);
            if (k8_hi - k8_lo == 8) {
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const int k8 = k8_lo + q;
                umma_tf32_ts(o_tmem, p_tmem + k8 * 8, v_base + k8 * 64, idesc_o, q > 0 ? 1u : started);
              }
              started = 1;
            } else {
              for (int k8 = k8_lo; k8 < k8_hi; ++k8) {
                umma_tf32_ts(o_tmem, p_tmem + k8 * 8, v_base + k8 * 64, idesc_o, started);
                started = 1;
              }
            }
            umma_commit(bar_ring_empty + 8 * rs);
            if (++rs == kRing) { rs = 0; r_ph ^= 1; }
          }
          if (!ok) break;
          umma_commit(bar_o_full);
          // P lives where the next tile's scores go: wait until both threads' P V MMAs have consumed it
          if (!(ok = mbar_wait(bar_o_full, t_ph, abort_flag, p.status, 2u))) break;
          t_ph ^= 1;
        }
      }
    }
  } else {
    // ------------------------------- softmax + output -------------------------------
    // Two warps per TMEM lane quarter: `half` 0 takes the even 32-column blocks of the row, half 1
    // the odd ones; row maximum and row sum are combined through shared memory, the pair meeting on
    // a named barrier of its own. For the output each half normalises and stores 32 of the 64 columns.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int pair_bar = 1 + quarter;  // named barrier ids 1..4 (0 is __syncthreads)
    uint32_t t_ph = 0;
    bool ok = true;
    for (int64_t item = blockIdx.x; item < p.items && ok; item += gridDim.x) {
      const int b = (int)(item / p.heads), h = (int)(item % p.heads);
      for (int mt = 0; mt < p.n_blocks; ++mt) {
        if (!(ok = mbar_wait(bar_s_full, t_ph, abort_flag, p.status, 8u))) break;
        tc_fence_after();
        float mx = -INFINITY;
        for (int c = half * 32; c < p.S; c += 64) {
          uint32_t v[32];
          tmem_ld32(lane_addr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) mx = fmaxf(mx, __uint_as_float(v[j]));
        }
        s_red[half][row_in_tile] = mx;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        mx = fmaxf(mx, s_red[half ^ 1][row_in_tile]);
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");  // both have read before s_red is reused
        const float off = mx * p.scale_log2e;
        float sum = 0.f;
        for (int ch = 0; ch < n_chunks; ++ch) {
          const int c_end = (ch + 1) * 128 < p.S ? (ch + 1) * 128 : p.S;
          for (int c = ch * 128 + half * 32; c < c_end; c += 64) {
            uint32_t v[32];
            tmem_ld32(lane_addr + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float e;
              asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(fmaf(__uint_as_float(v[j]), p.scale_log2e, -off)));
              sum += e;
              v[j] = __float_as_uint(e);
            }
            tmem_st32(lane_addr + c, v);
          }
          // every thread arrives once per 128-column group, whether or not it owned a block in it
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive(bar_p_full + 8 * ch);
        }
        s_red[half][row_in_tile] = sum;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        sum += s_red[half ^ 1][row_in_tile];
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        if (!(ok = mbar_wait(bar_o_full, t_ph, abort_flag, p.status, 8u))) break;
        tc_fence_after();
        const int row = mt * 128 + row_in_tile;
        const float inv = 1.0f / sum;
        float *orow = p.out + (int64_t)b * p.o_batch + (int64_t)row * p.o_row + (int64_t)h * p.o_head + half * 32;
        {
          uint32_t v[32];
          tmem_ld32(lane_addr + kOCol + half * 32, v);
          if (p.S > 64) {  // the second partial output exists once a key group has more than 64 keys
            uint32_t v2[32];
            tmem_ld32(lane_addr + kOCol2 + half * 32, v2);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(v2[j]));
          }
          tmem_ld_wait();
          tc_fence_before();
          mbar_arrive(bar_o_empty);  // the accumulators may be overwritten by the next tile
          if (row < p.S) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              float o[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(v[j + i]) * inv;
              asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(orow + j), "f"(o[0]), "f"(o[1]),
                           "f"(o[2]), "f"(o[3]), "f"(o[4]), "f"(o[5]), "f"(o[6]), "f"(o[7])
                           : "memory");
            }
          }
        }
        t_ph ^= 1;
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (s_abort) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}


// ---------------------------------------------------------------------------------------------
// Streaming variant: key / value blocks of 128 are consumed one at a time with a running row maximum
// and row sum (the softmax of the exported graph, evaluated block by block: P_j = exp(s - m_j) with
// m_j the exponent offset so far, O and the row sum rescaled by exp(m_{j-1} - m_j) when the offset moves),
// so TMEM use does not depend on the sequence length.
// ---------------------------------------------------------------------------------------------

struct BlkIter {
  int it, mt, j;  // this CTA's item counter, query tile, key block
  __device__ __forceinline__ void next(int nb) {
    if (++j == nb) { j = 0; if (++mt == nb) { mt = 0; ++it; } }
  }
};

// ---------------------------------------------------------------------------------------------
// Several MMA-issuing threads: one thread issuing every tcgen05.mma of a key block (8 for the scores, 16 for
// P V, ~90-130 clk each; measured with clock64()) needs ~3000 clk per block - more than the softmax warps
// (~1650) or the tensor core. Here warp 1 issues the scores and warps 10 and 11 the P V products
// (half the keys of a block each, into two partial output accumulators that are added at the end), the
// scores rotate through three 128-column TMEM buffers (so the score thread runs up to three blocks
// ahead of P V), and keys and values have rings of their own. The exponent offset follows the running
// maximum lazily (only when that has grown by more than 2^8), so rescaling O is rare.
//   s_full[3]  A -> softmax      p_full[3]  softmax (256) -> B      pv[3]  B -> A (buffer free), softmax
//   k_full/k_empty[3], v_full/v_empty[2], q_full/q_empty[2]: loads    o_empty  softmax (256) -> B
// ---------------------------------------------------------------------------------------------
constexpr int kThreads2 = 32 * 12;  // producer, issuer A, 8 softmax / output warps, issuers B1 and B2
constexpr int kOColA = 384, kOColB = 448;  // the two partial output accumulators (B1: first 64 keys of a block, B2: rest)

__global__ void __launch_bounds__(kThreads2, 1)
attention_stream_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t q_smem = smem_u32(smem);
  const uint32_t k_smem = q_smem + 2 * kBlkBytes;          // three key blocks (issuer A's ring)
  const uint32_t v_smem = k_smem + 3 * kBlkBytes;          // two value blocks (issuer B's ring)
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + 7 * (size_t)kBlkBytes);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_q_full = bar0, bar_q_empty = bar0 + 16, bar_k_full = bar0 + 32, bar_k_empty = bar0 + 56,
                 bar_v_full = bar0 + 80, bar_v_empty = bar0 + 96, bar_s_full = bar0 + 112, bar_p_full = bar0 + 136,
                 bar_pv = bar0 + 160, bar_o_empty = bar0 + 184;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ float s_red[2][128];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_q_full + 8 * i, 1);
      mbar_init(bar_q_empty + 8 * i, 1);
      mbar_init(bar_v_full + 8 * i, 1);
      mbar_init(bar_v_empty + 8 * i, 2);  // both P V issuers release a value block
    }
    for (int i = 0; i < 3; ++i) {
      mbar_init(bar_k_full + 8 * i, 1);
      mbar_init(bar_k_empty + 8 * i, 1);
      mbar_init(bar_s_full + 8 * i, 1);
      mbar_init(bar_p_full + 8 * i, 256);
      mbar_init(bar_pv + 8 * i, 2);       // both halves of P_g V_g
    }
    mbar_init(bar_o_empty, 256);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&s_tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int *abort_flag = &s_abort;
  const int nb = p.n_blocks;
  const int n_my = (int)((p.items - blockIdx.x + gridDim.x - 1) / gridDim.x);  // items of this CTA
  const int64_t G = (int64_t)n_my * nb * nb;                                    // blocks of this CTA

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    // Key blocks go to a ring of three (consumed by the score issuer, which runs up to three blocks ahead),
    // value blocks to a ring of two (consumed by the P V issuer): K_0 K_1 K_2, then V_g, K_{g+3} for every g.
    if (lane == 0) {
      int qs = 0;
      uint32_t q_ph = 0;
      bool ok = true;
      auto coords = [&](const BlkIter &x, int &b, int &h) {
        const int64_t item = blockIdx.x + (int64_t)x.it * gridDim.x;
        b = (int)(item / p.heads);
        h = (int)(item % p.heads);
      };
      auto load_k = [&](const BlkIter &x, int64_t g) {
        int b, h;
        coords(x, b, h);
        if (x.j == 0) {
          if (!(ok = mbar_wait(bar_q_empty + 8 * qs, q_ph ^ 1, abort_flag, p.status, 1u))) return;
          mbar_expect_tx(bar_q_full + 8 * qs, kBlkBytes);
          tma_load_4d(q_smem + qs * kBlkBytes, &map_q, bar_q_full + 8 * qs, 0, x.mt * 128, h, b);
          tma_load_4d(q_smem + qs * kBlkBytes + kBlkBytes / 2, &map_q, bar_q_full + 8 * qs, 32, x.mt * 128, h, b);
          if (++qs == 2) { qs = 0; q_ph ^= 1; }
        }
        const uint32_t slot = (uint32_t)(g % 3), full = bar_k_full + 8 * slot;
        if (!(ok = mbar_wait(bar_k_empty + 8 * slot, (uint32_t)((g / 3) & 1) ^ 1, abort_flag, p.status, 1u))) return;
        mbar_expect_tx(full, kBlkBytes);
        tma_load_4d(k_smem + slot * kBlkBytes, &map_k, full, 0, x.j * 128, h, b);
        tma_load_4d(k_smem + slot * kBlkBytes + kBlkBytes / 2, &map_k, full, 32, x.j * 128, h, b);
      };
      BlkIter kq{0, 0, 0}, v{0, 0, 0};
      int64_t gk = 0;
      for (; gk < 3 && gk < G && ok; ++gk) { load_k(kq, gk); kq.next(nb); }
      for (int64_t g = 0; g < G && ok; ++g) {
        int b, h;
        coords(v, b, h);
        const uint32_t slot = (uint32_t)(g & 1), full = bar_v_full + 8 * slot;
        if (!(ok = mbar_wait(bar_v_empty + 8 * slot, (uint32_t)((g >> 1) & 1) ^ 1, abort_flag, p.status, 1u))) break;
        mbar_expect_tx(full, kBlkBytes);
        tma_load_4d(v_smem + slot * kBlkBytes, &map_v, full, 0, v.j * 128, h, b);
        tma_load_4d(v_smem + slot * kBlkBytes + kBlkBytes / 2, &map_v, full, 32, v.j * 128, h, b);
        v.next(nb);
        if (gk < G) { load_k(kq, gk); kq.next(nb); ++gk; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- issuer A: scores -------------------------------
    // S_g = Q K_g^T into score buffer g % 3, as soon as P V_{g-3} has consumed what that buffer held.
    if (lane == 0) {
      int qs = 0;
      uint32_t q_ph = 0;
      const uint32_t idesc_full = make_idesc(128, false);
      const uint64_t kdesc0 = make_smem_desc(0, 16, 1024, kLayoutSw128);
      bool ok = true;
      BlkIter kq{0, 0, 0};
      for (int64_t g = 0; g < G && ok; ++g) {
        const uint32_t sb = (uint32_t)(g % 3), sp = (uint32_t)((g / 3) & 1);
        if (g >= 3) {
          if (!(ok = mbar_wait(bar_pv + 8 * sb, sp ^ 1, abort_flag, p.status, 2u))) break;  // completion g/3 - 1
        }
        if (kq.j == 0) {
          if (!(ok = mbar_wait(bar_q_full + 8 * qs, q_ph, abort_flag, p.status, 2u))) break;
        }
        if (!(ok = mbar_wait(bar_k_full + 8 * sb, sp, abort_flag, p.status, 2u))) break;
        tc_fence_after();
        const int n_len = p.S - kq.j * 128;
        const uint32_t idesc_s = n_len >= 128 ? idesc_full : make_idesc(n_len, false);
        const uint64_t a_base = kdesc0 + ((q_smem + qs * kBlkBytes) >> 4);
        const uint64_t b_base = kdesc0 + ((k_smem + sb * kBlkBytes) >> 4);
        const uint32_t d_tmem = tmem_base + sb * 128;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          constexpr uint32_t kHalf = (kBlkBytes / 2) >> 4;
          const uint32_t off = (ks >> 2) * kHalf + (ks & 3) * 2;
          umma_tf32(d_tmem, a_base + off, b_base + off, idesc_s, ks > 0 ? 1u : 0u);
        }
        umma_commit(bar_k_empty + 8 * sb);
        umma_commit(bar_s_full + 8 * sb);
        if (kq.j == nb - 1) {
          umma_commit(bar_q_empty + 8 * qs);
          if (++qs == 2) { qs = 0; q_ph ^= 1; }
        }
        kq.next(nb);
      }
    }
  } else if (warp >= 10) {
    // ------------------------------- issuers B1 / B2: O += P_g V_g -------------------------------
    // Warp 10 multiplies the first 64 keys of every block into accumulator A, warp 11 the remaining keys into
    // accumulator B (two threads issue the N = 64 instructions faster than one; the output is A + B).
    if (lane == 0) {
      const int second = warp - 10;
      const uint32_t o_tmem = tmem_base + (second ? kOColB : kOColA);
      const uint32_t idesc_o = make_idesc(kD, true);
      const uint64_t vdesc0 = make_smem_desc(0, kBlkBytes / 2, 512, kLayoutSw128Base32);
      bool ok = true;
      BlkIter pv{0, 0, 0};
      int64_t tile = 0;
      uint32_t started = 0;  // 0 until this accumulator has received its first product of the tile
      for (int64_t g = 0; g < G && ok; ++g) {
        const uint32_t sb = (uint32_t)(g % 3), sp = (uint32_t)((g / 3) & 1), vs = (uint32_t)(g & 1);
        if (pv.j == 0) {  // the previous tile's output must have been read before O is overwritten
          if (!(ok = mbar_wait(bar_o_empty, (uint32_t)(tile & 1) ^ 1, abort_flag, p.status, 4u))) break;
          ++tile;
          started = 0;
        }
        if (!(ok = mbar_wait(bar_p_full + 8 * sb, sp, abort_flag, p.status, 4u))) break;
        if (!(ok = mbar_wait(bar_v_full + 8 * vs, (uint32_t)((g >> 1) & 1), abort_flag, p.status, 4u))) break;
        tc_fence_after();
        const uint64_t v_base = vdesc0 + ((v_smem + vs * kBlkBytes) >> 4);
        const uint32_t p_tmem = tmem_base + sb * 128;
        const int k_len = p.S - pv.j * 128 < 128 ? p.S - pv.j * 128 : 128;
        const int k8_lo = second ? 8 : 0, k8_hi = second ? k_len / 8 : (k_len / 8 < 8 ? k_len / 8 : 8);
        if (k8_hi - k8_lo == 8) {
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int k8 = k8_lo + q;
            umma_tf32_ts(o_tmem, p_tmem + k8 * 8, v_base + k8 * 64, idesc_o, q > 0 ? 1u : started);
          }
          started = 1;
        } else {
          for (int k8 = k8_lo; k8 < k8_hi; ++k8) {
            umma_tf32_ts(o_tmem, p_tmem + k8 * 8, v_base + k8 * 64, idesc_o, started);
            started = 1;
          }
        }
        umma_commit(bar_v_empty + 8 * vs);
        umma_commit(bar_pv + 8 * sb);
        pv.next(nb);
      }
    }
  } else {
    // ------------------------------- softmax + output -------------------------------
    // Two warps per TMEM lane quarter, one score row per thread: `half` 0 owns columns [0, 64) of every
    // 128-column block, half 1 columns [64, 128); for the output each owns 32 of the 64 columns.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int pair_bar = 1 + quarter;
    const float c = p.scale_log2e;
    bool ok = true;
    BlkIter bi{0, 0, 0};
    float m_run = -INFINITY, l_run = 0.f;
    for (int64_t g = 0; g < G && ok; ++g) {
      const uint32_t sb = (uint32_t)(g % 3), sp = (uint32_t)((g / 3) & 1);
      const uint32_t s_addr = lane_addr + sb * 128 + half * 64;
      const int k_len = p.S - bi.j * 128 < 128 ? p.S - bi.j * 128 : 128;
      const int n_mine = k_len - half * 64 >= 64 ? 64 : (k_len - half * 64 > 0 ? k_len - half * 64 : 0);  // 0, 32 or 64
      if (!(ok = mbar_wait(bar_s_full + 8 * sb, sp, abort_flag, p.status, 8u))) break;
      tc_fence_after();
      uint32_t v0[32], v1[32];
      if (n_mine >= 32) tmem_ld32(s_addr, v0);
      if (n_mine == 64) tmem_ld32(s_addr + 32, v1);
      tmem_ld_wait();
      float m_loc = -INFINITY;
      if (n_mine >= 32) {
#pragma unroll
        for (int i = 0; i < 32; ++i) m_loc = fmaxf(m_loc, __uint_as_float(v0[i]));
      }
      if (n_mine == 64) {
#pragma unroll
        for (int i = 0; i < 32; ++i) m_loc = fmaxf(m_loc, __uint_as_float(v1[i]));
      }
      s_red[half][row_in_tile] = m_loc;
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      const float m_blk = fmaxf(m_loc, s_red[half ^ 1][row_in_tile]);
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      // The exponent offset only follows the running maximum when that has grown by more than 2^8 (in the
      // exp2 domain): P then stays below 256 instead of 1, which fp32 / TF32 hold just as well, and the
      // rescaling of O - with its wait for the previous block's P V - becomes rare.
      const bool grow = bi.j == 0 || (m_blk - m_run) * c > 8.0f;
      const float m_new = grow ? m_blk : m_run;
      float alpha = 1.0f;  // exp((m_run - m_new) * scale): the factor by which earlier blocks' terms shrink
      if (grow) asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(alpha) : "f"((m_run - m_new) * c));
      if (bi.j == 0) alpha = 0.f;
      const float off = m_new * c;
      float sum = 0.f;
      if (n_mine >= 32) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e;
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(fmaf(__uint_as_float(v0[i]), c, -off)));
          sum += e;
          v0[i] = __float_as_uint(e);
        }
        tmem_st32(s_addr, v0);
      }
      if (n_mine == 64) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e;
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(fmaf(__uint_as_float(v1[i]), c, -off)));
          sum += e;
          v1[i] = __float_as_uint(e);
        }
        tmem_st32(s_addr + 32, v1);
      }
      l_run = l_run * alpha + sum;
      m_run = m_new;
      if (bi.j > 0 && __any_sync(0xffffffffu, grow)) {
        // O holds sum_{i<j} P_i V_i relative to the old offset: wait for P_{j-1} V_{j-1}, then rescale this
        // thread's 32 output columns (rows of the warp that kept their offset multiply by 1)
        if (!(ok = mbar_wait(bar_pv + 8 * (uint32_t)((g - 1) % 3), (uint32_t)(((g - 1) / 3) & 1), abort_flag, p.status,
                             8u)))
          break;
        tc_fence_after();
#pragma unroll 1
        for (int acc = 0; acc < (p.S > 64 ? 2 : 1); ++acc) {
          uint32_t o[32];
          const uint32_t o_addr = lane_addr + (acc ? kOColB : kOColA) + half * 32;
          tmem_ld32(o_addr, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(o_addr, o);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar_p_full + 8 * sb);

      if (bi.j == nb - 1) {
        // ---- the tile's last block: normalise and store once its P V has been accumulated ----
        s_red[half][row_in_tile] = l_run;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        const float l_tot = l_run + s_red[half ^ 1][row_in_tile];
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        if (!(ok = mbar_wait(bar_pv + 8 * sb, sp, abort_flag, p.status, 8u))) break;
        tc_fence_after();
        const int64_t item = blockIdx.x + (int64_t)bi.it * gridDim.x;
        const int b = (int)(item / p.heads), h = (int)(item % p.heads);
        const int row = bi.mt * 128 + row_in_tile;
        const float inv = 1.0f / l_tot;
        float *orow = p.out + (int64_t)b * p.o_batch + (int64_t)row * p.o_row + (int64_t)h * p.o_head + half * 32;
        uint32_t o[32];
        tmem_ld32(lane_addr + kOColA + half * 32, o);
        if (p.S > 64) {  // accumulator B exists once a block has more than 64 keys
          uint32_t o2[32];
          tmem_ld32(lane_addr + kOColB + half * 32, o2);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) + __uint_as_float(o2[i]));
        }
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(bar_o_empty);
        if (row < p.S) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            float r[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) r[q] = __uint_as_float(o[i + q]) * inv;
            asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(orow + i), "f"(r[0]), "f"(r[1]),
                         "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]), "f"(r[7])
                         : "memory");
          }
        }
        m_run = -INFINITY;
        l_run = 0.f;
      }
      bi.next(nb);
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (s_abort) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
  }
  if (warp == 1) {
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
  p.items = d.batch * d.heads;
  p.scale_log2e = d.scale * 1.4426950408889634f;
  p.out = out;
  p.o_batch = d.o_batch;
  p.o_row = d.o_row;
  p.o_head = d.o_head;
  p.status = device_status_ptr();
  if (!p.status) return fail(B200_ECUDA, "attention: device status word unavailable");
  const int smem = (2 + kRing) * kBlkBytes + 1024 + 256;
  if (cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return fail(B200_ECUDA, "attention: cannot set dynamic shared memory to %d", smem);
  const int64_t grid = p.items < kNumSMs ? p.items : kNumSMs;
  // Rows of up to 384 scores stay resident in TMEM (two-pass softmax; measured 264-270 against 249-254 TFLOP/s for
  // the streaming kernel at S = 384); longer rows stream.
#ifndef B200_ATTENTION_ALWAYS_STREAM  // build-time switch for comparing the two kernels on sequences both can run
  if (d.seq <= kMaxS)
#else
  if (false)
#endif
  {
    attention_tc_kernel<<<(unsigned)grid, kThreads, smem, st>>>(mq, mk, mv, p);
    return check_launch("attention_tc");
  }
  if (cudaFuncSetAttribute(attention_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return fail(B200_ECUDA, "attention: cannot set dynamic shared memory to %d", smem);
  attention_stream_kernel<<<(unsigned)grid, kThreads2, smem, st>>>(mq, mk, mv, p);
  return check_launch("attention_stream");
}

}  // namespace b200
