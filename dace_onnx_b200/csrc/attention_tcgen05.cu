// Fused attention for sm_100a: softmax(Q K^T * scale) V per (batch, head) without materialising
// the [S, S] score matrix in HBM. Replaces the node pattern MatMul -> Mul(const) -> Softmax ->
// MatMul of the exported BERT graph (TF32 tensor-core mode).
//
// One persistent CTA per SM walks (batch, head) items. K and V of the item stay in shared memory
// (K as the K-major B operand of Q K^T, V as the MN-major B operand of P V); the query tiles of
// 128 rows stream through a single Q buffer. Per query tile:
//   warp 1 issues Q K^T into TMEM columns [0, S)            (tcgen05.mma kind::tf32, A and B in smem)
//   warps 2-5 (one score row per thread) read the row from TMEM, take its maximum, overwrite it in
//             place with P = exp2((s - max) * scale * log2 e) and sum P          (tcgen05.ld / st)
//   warp 1 issues P V with the A operand read from TMEM into columns [448, 512), 128 key columns
//             at a time as soon as the softmax warps have published them
//   warps 2-5 read the 64 output columns, divide by the row sum and store [row, head*64 .. +64).
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

constexpr int kD = 64;            // head dimension
constexpr int kQBytes = 128 * kD * 4;   // 32 KiB: two k-blocks of [128 rows][128 B]
constexpr int kOCol = 448;        // TMEM column of the output accumulator
constexpr int kMaxS = 384;

struct AttnParams {
  int S, Sp;          // sequence length; Sp = S rounded up to 128 (row capacity of the K / V buffers)
  int heads;
  int m_tiles;
  int64_t items;      // batch * heads
  float scale_log2e;
  float *out;
  int64_t o_batch, o_row, o_head;  // element strides of the output
  unsigned *status;
};

__global__ void __launch_bounds__(192, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t q_smem = smem_u32(smem);
  const uint32_t kblk_bytes = (uint32_t)p.Sp * 128;  // one 32-wide slice of K or V: [Sp rows][128 B]
  const uint32_t k_smem = q_smem + kQBytes;
  const uint32_t v_smem = k_smem + 2 * kblk_bytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kQBytes + 4 * (size_t)kblk_bytes);
  const uint32_t bar_kv_full = smem_u32(bars), bar_kv_empty = bar_kv_full + 8, bar_q_full = bar_kv_full + 16,
                 bar_q_empty = bar_kv_full + 24, bar_s_full = bar_kv_full + 32, bar_o_full = bar_kv_full + 40,
                 bar_o_empty = bar_kv_full + 48, bar_p_full = bar_kv_full + 56;  // p_full[0..3]
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(bar_kv_full, 1);
    mbar_init(bar_kv_empty, 1);
    mbar_init(bar_q_full, 1);
    mbar_init(bar_q_empty, 1);
    mbar_init(bar_s_full, 1);
    mbar_init(bar_o_full, 1);
    mbar_init(bar_o_empty, 128);
    for (int c = 0; c < 4; ++c) mbar_init(bar_p_full + 8 * c, 128);
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
  const int n_chunks = (p.S + 127) / 128;  // 128-column groups of P handed to the P V MMAs

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      uint32_t kv_ph = 0, q_ph = 0;
      bool ok = true;
      for (int64_t item = blockIdx.x; item < p.items && ok; item += gridDim.x) {
        const int b = (int)(item / p.heads), h = (int)(item % p.heads);
        if (!(ok = mbar_wait(bar_kv_empty, kv_ph ^ 1, abort_flag, p.status, 1u))) break;
        mbar_expect_tx(bar_kv_full, 4 * kblk_bytes);
        for (int kb = 0; kb < 2; ++kb)
          for (int r0 = 0; r0 < p.Sp; r0 += 128) {
            tma_load_4d(k_smem + kb * kblk_bytes + r0 * 128, &map_k, bar_kv_full, kb * 32, r0, h, b);
            tma_load_4d(v_smem + kb * kblk_bytes + r0 * 128, &map_v, bar_kv_full, kb * 32, r0, h, b);
          }
        kv_ph ^= 1;
        for (int mt = 0; mt < p.m_tiles; ++mt) {
          if (!(ok = mbar_wait(bar_q_empty, q_ph ^ 1, abort_flag, p.status, 1u))) break;
          mbar_expect_tx(bar_q_full, kQBytes);
          tma_load_4d(q_smem, &map_q, bar_q_full, 0, mt * 128, h, b);
          tma_load_4d(q_smem + kQBytes / 2, &map_q, bar_q_full, 32, mt * 128, h, b);
          q_ph ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      uint32_t kv_ph = 0, t_ph = 0;  // t_ph: phase of the per-tile barriers (q_full, o_empty, p_full, o_full)
      const uint32_t idesc_o = make_idesc(kD, true);
      bool ok = true;
      for (int64_t item = blockIdx.x; item < p.items && ok; item += gridDim.x) {
        if (!(ok = mbar_wait(bar_kv_full, kv_ph, abort_flag, p.status, 2u))) break;
        kv_ph ^= 1;
        for (int mt = 0; mt < p.m_tiles && ok; ++mt) {
          if (!(ok = mbar_wait(bar_q_full, t_ph, abort_flag, p.status, 2u))) break;
          tc_fence_after();
          // S = Q K^T: N is issued in pieces of at most 256 columns
          for (int n0 = 0; n0 < p.S; n0 += 256) {
            const int n_len = p.S - n0 < 256 ? p.S - n0 : 256;
            const uint32_t idesc_s = make_idesc(n_len, false);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const int kb = ks >> 2, kk = ks & 3;
              const uint64_t a = make_smem_desc(q_smem + kb * (kQBytes / 2) + kk * 32, 16, 1024, kLayoutSw128);
              const uint64_t bd = make_smem_desc(k_smem + kb * kblk_bytes + n0 * 128 + kk * 32, 16, 1024, kLayoutSw128);
              umma_tf32(tmem_base + n0, a, bd, idesc_s, ks > 0 ? 1u : 0u);
            }
          }
          umma_commit(bar_q_empty);  // Q buffer reusable
          umma_commit(bar_s_full);   // scores ready for the softmax warps
          // O = P V, A operand (P) from TMEM; the previous tile's O must have been read out
          if (!(ok = mbar_wait(bar_o_empty, t_ph ^ 1, abort_flag, p.status, 2u))) break;
          for (int c = 0; c < n_chunks && ok; ++c) {
            if (!(ok = mbar_wait(bar_p_full + 8 * c, t_ph, abort_flag, p.status, 4u))) break;
            tc_fence_after();
            const int k_end = (c + 1) * 128 < p.S ? (c + 1) * 128 : p.S;
            for (int k0 = c * 128; k0 < k_end; k0 += 8) {
              // 8 key rows of V: [k0, k0+8) x 64, two 32-column chunks kblk_bytes apart
              const uint64_t bd = make_smem_desc(v_smem + k0 * 128, kblk_bytes, 512, kLayoutSw128Base32);
              umma_tf32_ts(tmem_base + kOCol, tmem_base + k0, bd, idesc_o, k0 > 0 ? 1u : 0u);
            }
          }
          if (!ok) break;
          umma_commit(bar_o_full);
          if (mt + 1 == p.m_tiles) umma_commit(bar_kv_empty);  // K / V buffers reusable
          // P lives where the next tile's scores go: wait until the P V MMAs have consumed it
          if (!(ok = mbar_wait(bar_o_full, t_ph, abort_flag, p.status, 2u))) break;
          t_ph ^= 1;
        }
      }
    }
  } else {
    // ------------------------------- softmax + output (one row per thread) -------------------------------
    const int quarter = warp & 3;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    uint32_t t_ph = 0;
    bool ok = true;
    for (int64_t item = blockIdx.x; item < p.items && ok; item += gridDim.x) {
      const int b = (int)(item / p.heads), h = (int)(item % p.heads);
      for (int mt = 0; mt < p.m_tiles; ++mt) {
        if (!(ok = mbar_wait(bar_s_full, t_ph, abort_flag, p.status, 8u))) break;
        tc_fence_after();
        float mx = -INFINITY;
        for (int c = 0; c < p.S; c += 32) {
          uint32_t v[32];
          tmem_ld32(lane_addr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) mx = fmaxf(mx, __uint_as_float(v[j]));
        }
        const float off = mx * p.scale_log2e;
        float sum = 0.f;
        for (int c = 0; c < p.S; c += 32) {
          uint32_t v[32];
          tmem_ld32(lane_addr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float e = exp2f(fmaf(__uint_as_float(v[j]), p.scale_log2e, -off));
            sum += e;
            v[j] = __float_as_uint(e);
          }
          tmem_st32(lane_addr + c, v);
          if (((c + 32) & 127) == 0 || c + 32 >= p.S) {
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(bar_p_full + 8 * (c >> 7));
          }
        }
        if (!(ok = mbar_wait(bar_o_full, t_ph, abort_flag, p.status, 8u))) break;
        tc_fence_after();
        const int row = mt * 128 + quarter * 32 + lane;
        const float inv = 1.0f / sum;
        float *orow = p.out + (int64_t)b * p.o_batch + (int64_t)row * p.o_row + (int64_t)h * p.o_head;
#pragma unroll
        for (int c = 0; c < kD; c += 32) {
          uint32_t v[32];
          tmem_ld32(lane_addr + kOCol + c, v);
          tmem_ld_wait();
          if (c + 32 >= kD) {
            tc_fence_before();
            mbar_arrive(bar_o_empty);  // the accumulator may be overwritten by the next tile
          }
          if (row < p.S) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              float o[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(v[j + i]) * inv;
              asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(orow + c + j), "f"(o[0]), "f"(o[1]),
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
  if (d.head_dim != kD || d.seq < 32 || d.seq > kMaxS || d.seq % 32 != 0) return false;
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
  p.Sp = (int)((d.seq + 127) / 128 * 128);
  p.heads = (int)d.heads;
  p.m_tiles = p.Sp / 128;
  p.items = d.batch * d.heads;
  p.scale_log2e = d.scale * 1.4426950408889634f;
  p.out = out;
  p.o_batch = d.o_batch;
  p.o_row = d.o_row;
  p.o_head = d.o_head;
  p.status = device_status_ptr();
  if (!p.status) return fail(B200_ECUDA, "attention: device status word unavailable");
  const int smem = kQBytes + 4 * p.Sp * 128 + 1024 + 128;
  if (cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return fail(B200_ECUDA, "attention: cannot set dynamic shared memory to %d", smem);
  const int64_t grid = p.items < kNumSMs ? p.items : kNumSMs;
  attention_tc_kernel<<<(unsigned)grid, 192, smem, st>>>(mq, mk, mv, p);
  return check_launch("attention_tc");
}

}  // namespace b200
