// Tensor-core GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma (kind::tf32) -> TMEM -> epilogue.
//
// One persistent CTA per SM walks a static list of 128 x BN output tiles. Inside a CTA the warps
// are specialised:
//   warp 0      TMA producer: one lane issues cp.async.bulk.tensor loads of the A and B k-blocks
//               (128B-swizzled, 32 fp32 of K per block) into a ring of shared-memory stages;
//   warp 1      MMA issuer: allocates TMEM, one lane issues tcgen05.mma for each 8-wide k-step
//               and commits stage release / accumulator-ready events to mbarriers;
//   next 8 or 16 warps: epilogue: tcgen05.ld the fp32 accumulator (row = TMEM lane, one row per thread,
//               two or four warps per lane quarter), apply the fused epilogue (bias / ReLU / erf-Gelu /
//               residual / scale) and store with 256-bit vector stores, each thread writing whole
//               32-byte sectors of its row (128-bit / scalar stores when Y is less aligned);
//   last 8 warps (3xTF32 mode only) split warps: split each landed stage into hi = tf32(x) and
//               lo = tf32(x - hi) -- A into TMEM (the MMAs then read A from TMEM), B in shared
//               memory -- so that the issuer can run lo*hi + hi*lo + hi*hi into the same fp32
//               accumulator (fp32-accurate products).
// Two TMEM accumulators alternate so that the epilogue of tile i overlaps the MMAs of tile i+1.
//
// Every mbarrier wait is bounded by a cycle budget; on expiry the CTA sets a bit in the device
// status word, all roles leave their loops, TMEM is released and the kernel returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <string.h>

#include <atomic>

#include "common.cuh"
#include "contract.cuh"
#include "tc_common.cuh"

namespace b200 {
using namespace tc;
namespace {

constexpr int BM = 128;
constexpr int BK = 32;                       // fp32 elements per k-block = one 128-byte swizzle row
constexpr int UMMA_K = 8;                    // K of one kind::tf32 instruction
constexpr int A_STAGE_BYTES = BM * BK * 4;   // 16 KiB
// Geometry of a stride-1 convolution run as an implicit GEMM: rows of the GEMM are output pixels,
// grouped in 8x8 blocks (two blocks per 128-row tile); K runs over (kh, kw, 32-channel block).
struct ConvGeom {
  int KW, pad_h, pad_w;
  int OH, OW;
  int blocks_w, blocks_per_img;  // 8x8 output blocks per row / per image
  int cblocks;                   // 32-channel blocks per filter tap
  int64_t total_blocks;          // images * blocks_per_img
};

struct GemmParams {
  ConvGeom cv;
  int64_t M, N;
  int num_kb;
  int num_m_tiles, num_n_tiles;
  int64_t num_tiles;
  int64_t num_tiles_batch;  // number of batch matrices (pair kernel: tiles = m pairs x n tiles x this)
  int batch_inner;
  int a_bi, a_bo, b_bi, b_bo;  // 1 when the operand advances with that batch index, 0 when broadcast
  int vec;                     // widest aligned access to Y / residual rows: 8, 4 or 1 floats
  int64_t ldy, y_stride_outer, y_stride_inner;
  int epilogue;
  float scale;
  const float *bias;
  const float *residual;
  float *Y;
  unsigned *status;
};

// k-blocks per in-core accumulation chunk in 3xTF32 mode (4 x 32 = 128 values of K, 48 MMAs).
constexpr int kSplitChunkKb = 4;

__device__ __forceinline__ void ld_global_v8(const float *p, float *v) {
  asm volatile("ld.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7])
               : "l"(p));
}
__device__ __forceinline__ void st_global_v8(float *p, const float *v) {
  asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
               : "memory");
}

// Fused epilogue and store of 32 consecutive columns [n0, n0+32) of output row m, held in registers
// by one thread. Each thread owns 128 contiguous bytes of its row; with 32-byte vector accesses every
// store instruction writes whole 32-byte sectors (vec == 8), else 16-byte or scalar accesses.
// `bias_s`: when not null, the 32 bias values of these columns staged in shared memory (zero past N), read as
// broadcast 128-bit loads instead of global loads whose latency would serialise the store phase.
template <int EPI>
__device__ __forceinline__ void finish_row32_t(const GemmParams &p, float *v, int64_t m, int64_t row_off, int64_t n0,
                                               const float *bias_s = nullptr) {
  constexpr bool kBias = EPI == B200_EPI_BIAS || EPI == B200_EPI_BIAS_RELU || EPI == B200_EPI_BIAS_GELU ||
                         EPI == B200_EPI_BIAS_RESIDUAL;
  constexpr bool kResidual = EPI == B200_EPI_BIAS_RESIDUAL;
  if (m >= p.M || n0 >= p.N) return;
  const bool full = n0 + 32 <= p.N;
  float *yrow = p.Y + row_off + n0;
  const float *rrow = kResidual ? p.residual + row_off + n0 : nullptr;
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    float b[8], r[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) b[i] = r[i] = 0.f;
    if (kBias) {
      if (bias_s) {
        const float4 b0 = *reinterpret_cast<const float4 *>(bias_s + j);
        const float4 b1 = *reinterpret_cast<const float4 *>(bias_s + j + 4);
        b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w; b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
      } else if (full) {
        const float4 b0 = __ldg(reinterpret_cast<const float4 *>(p.bias + n0 + j));
        const float4 b1 = __ldg(reinterpret_cast<const float4 *>(p.bias + n0 + j + 4));
        b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w; b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (n0 + j + i < p.N) b[i] = __ldg(p.bias + n0 + j + i);
      }
    }
    if (kResidual) {
      if (full && p.vec == 8) {
        ld_global_v8(rrow + j, r);
      } else if (full && p.vec == 4) {
        const float4 r0 = *reinterpret_cast<const float4 *>(rrow + j);
        const float4 r1 = *reinterpret_cast<const float4 *>(rrow + j + 4);
        r[0] = r0.x; r[1] = r0.y; r[2] = r0.z; r[3] = r0.w; r[4] = r1.x; r[5] = r1.y; r[6] = r1.z; r[7] = r1.w;
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (n0 + j + i < p.N) r[i] = rrow[j + i];
      }
    }
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = apply_epilogue_t<EPI>(v[j + i], b[i], r[i], p.scale);
    if (full && p.vec == 8) {
      st_global_v8(yrow + j, o);
    } else if (full && p.vec == 4) {
      *reinterpret_cast<float4 *>(yrow + j) = make_float4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<float4 *>(yrow + j + 4) = make_float4(o[4], o[5], o[6], o[7]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (n0 + j + i < p.N) yrow[j + i] = o[i];
    }
  }
}

// The epilogue kind is uniform for the launch: choose the specialised body once per 32x32 block.
__device__ __forceinline__ void finish_row32(const GemmParams &p, float *v, int64_t m, int64_t row_off, int64_t n0,
                                             const float *bias_s = nullptr) {
  switch (p.epilogue) {
    case B200_EPI_BIAS: finish_row32_t<B200_EPI_BIAS>(p, v, m, row_off, n0, bias_s); break;
    case B200_EPI_BIAS_RELU: finish_row32_t<B200_EPI_BIAS_RELU>(p, v, m, row_off, n0, bias_s); break;
    case B200_EPI_BIAS_GELU: finish_row32_t<B200_EPI_BIAS_GELU>(p, v, m, row_off, n0, bias_s); break;
    case B200_EPI_BIAS_RESIDUAL: finish_row32_t<B200_EPI_BIAS_RESIDUAL>(p, v, m, row_off, n0, bias_s); break;
    case B200_EPI_SCALE: finish_row32_t<B200_EPI_SCALE>(p, v, m, row_off, n0); break;
    default: finish_row32_t<B200_EPI_NONE>(p, v, m, row_off, n0); break;
  }
}

// Convolution epilogue for 32 output channels [n0, n0+32) of one output pixel: bias / ReLU, then
// NCHW stores. For a fixed channel the 32 lanes of a warp hold 4 rows x 8 consecutive pixels, i.e.
// four whole 32-byte sectors per store instruction.
template <int EPI>
__device__ __forceinline__ void finish_pixel32_t(const GemmParams &p, const float *v, int64_t pix_off,
                                                 int64_t chan_stride, int64_t n0) {
  float *y = p.Y + pix_off + n0 * chan_stride;
  const bool full = n0 + 32 <= p.N;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    if (full || n0 + j < p.N) {
      const float b = (EPI != B200_EPI_NONE) ? __ldg(p.bias + n0 + j) : 0.f;
      y[j * chan_stride] = apply_epilogue_t<EPI>(v[j], b, 0.f, 1.f);
    }
  }
}
__device__ __forceinline__ void finish_pixel32(const GemmParams &p, const float *v, bool valid, int64_t pix_off,
                                               int64_t chan_stride, int64_t n0) {
  if (!valid || n0 >= p.N) return;
  switch (p.epilogue) {
    case B200_EPI_BIAS: finish_pixel32_t<B200_EPI_BIAS>(p, v, pix_off, chan_stride, n0); break;
    case B200_EPI_BIAS_RELU: finish_pixel32_t<B200_EPI_BIAS_RELU>(p, v, pix_off, chan_stride, n0); break;
    default: finish_pixel32_t<B200_EPI_NONE>(p, v, pix_off, chan_stride, n0); break;
  }
}

template <int BN, bool SPLIT3>
struct Cfg {
  static constexpr int kBStageBytes = BN * BK * 4;
  // 3xTF32: stage = [A raw | B -> B_hi in place | B_lo]; A's hi / lo halves live in TMEM, 64 columns
  // per stage behind the two accumulators, which bounds the stage count: 2*BN + 64*stages <= 512.
  static constexpr int kStageBytes = A_STAGE_BYTES + kBStageBytes * (SPLIT3 ? 2 : 1);
  static constexpr int kStagesSmem = (192 * 1024) / kStageBytes > 8 ? 8 : (192 * 1024) / kStageBytes;
  static constexpr int kStagesTmem = (512 - 2 * BN) / 64;
  static constexpr int kStages = (SPLIT3 && kStagesTmem < kStagesSmem) ? kStagesTmem : kStagesSmem;
  static constexpr int kTmemCols = SPLIT3 ? 512 : (2 * BN < 32 ? 32 : 2 * BN);  // two accumulators (+ A halves)
  static constexpr int kASplitCol0 = 2 * BN;  // first TMEM column of the A hi/lo stages
  // Epilogue warps: four per 64 accumulator columns, i.e. 2 (BN=64), 2 (BN=128, 3xTF32 keeps its
  // column sums in registers), 4 warps per TMEM lane quarter for the wide TF32 tiles, whose erf-Gelu
  // epilogue would otherwise take as long as the tile's MMAs.
  static constexpr int kWarpsPerQuarter = (BN >= 128 && !SPLIT3) ? 4 : 2;
  static constexpr int kEpilogueWarps = 4 * kWarpsPerQuarter;
  static constexpr int kSplitWarp0 = 2 + kEpilogueWarps;
  static constexpr int kSplitWarps = SPLIT3 ? 8 : 0;  // two per TMEM lane quarter
  static constexpr int kThreads = 32 * (2 + kEpilogueWarps + kSplitWarps);
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static constexpr int kColsPerWarp = BN / kWarpsPerQuarter;
};

// BF16: A and B are bf16 (64 values of K per 128-byte row, kind::f16 MMAs with K = 16); only with K-major B,
// without SPLIT3 / CONV. Tiles, stages and descriptors have the same byte geometry as the TF32 form.
template <int BN, bool B_MN, bool SPLIT3, bool CONV, bool BF16 = false>
__global__ void __launch_bounds__(Cfg<BN, SPLIT3>::kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const GemmParams p) {
  using C = Cfg<BN, SPLIT3>;
  constexpr int kStages = C::kStages;
  constexpr int BKE = BF16 ? 64 : BK;  // elements of K per k-block (one 128-byte row)
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: required by the 128-byte swizzle atoms the descriptors address.
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kStages * C::kStageBytes);
  // barrier layout: full[kStages] empty[kStages] split[kStages] tmem_full[2] tmem_empty[2]
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * kStages;
  const uint32_t bar_split = bar_empty + 8 * kStages;
  const uint32_t bar_tfull = bar_split + 8 * kStages;
  const uint32_t bar_tempty = bar_tfull + 16;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
      mbar_init(bar_split + 8 * s, 32 * (C::kSplitWarps > 0 ? C::kSplitWarps : 1));
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, C::kEpilogueWarps * 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&s_tmem_base), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int *abort_flag = &s_abort;

  auto stage_a = [&](int s) { return smem_base + s * C::kStageBytes; };
  auto stage_b = [&](int s) { return smem_base + s * C::kStageBytes + A_STAGE_BYTES; };

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      for (int64_t tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
        const int n_t = (int)(tile % p.num_n_tiles);
        const int64_t r = tile / p.num_n_tiles;
        const int m_t = (int)(r % p.num_m_tiles);
        const int64_t batch = r / p.num_m_tiles;
        const int bo = (int)(batch / p.batch_inner), bi = (int)(batch % p.batch_inner);
        // convolution: the two 8x8 output blocks of this tile, decomposed once per tile (integer
        // division is slow and this thread is alone on the critical path of every load)
        int cv_img[2] = {0, 0}, cv_x[2] = {0, 0}, cv_y[2] = {0, 0};
        if (CONV) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int64_t blk = 2 * (int64_t)m_t + h;
            cv_img[h] = (int)(blk / p.cv.blocks_per_img);
            const int rem = (int)(blk - (int64_t)cv_img[h] * p.cv.blocks_per_img);
            const int by = rem / p.cv.blocks_w;
            cv_y[h] = by * 8 - p.cv.pad_h;
            cv_x[h] = (rem - by * p.cv.blocks_w) * 8 - p.cv.pad_w;
          }
        }
        int cv_kh = 0, cv_kw = 0, cv_cb = 0;  // filter tap and channel block of the current k-block
        bool ok = true;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!(ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 1u))) break;
          mbar_expect_tx(bar_full + 8 * s, A_STAGE_BYTES + C::kBStageBytes);
          if (CONV) {
            // The A rows are the input pixels under tap (kh, kw) for the two output blocks.
            // Coordinates left of / above the image (the zero padding) and blocks past the last
            // image are filled with zeros by the TMA unit.
#pragma unroll
            for (int h = 0; h < 2; ++h)
              tma_load_4d(stage_a(s) + h * (A_STAGE_BYTES / 2), &map_a, bar_full + 8 * s, cv_cb * BK, cv_x[h] + cv_kw,
                          cv_y[h] + cv_kh, cv_img[h]);
            if (++cv_cb == p.cv.cblocks) {
              cv_cb = 0;
              if (++cv_kw == p.cv.KW) { cv_kw = 0; ++cv_kh; }
            }
          } else {
            tma_load_4d(stage_a(s), &map_a, bar_full + 8 * s, kb * BKE, m_t * BM, bi * p.a_bi, bo * p.a_bo);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 32; ++j)
              tma_load_4d(stage_b(s) + j * (BK * 128), &map_b, bar_full + 8 * s, n_t * BN + 32 * j, kb * BK,
                          bi * p.b_bi, bo * p.b_bo);
          } else {
            tma_load_4d(stage_b(s), &map_b, bar_full + 8 * s, kb * BKE, n_t * BN, bi * p.b_bi, bo * p.b_bo);
          }
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    // The K loop is cut into chunks; each chunk accumulates into its own TMEM buffer (the two
    // buffers alternate). In TF32 mode one chunk is the whole K. In 3xTF32 mode a chunk is
    // kSplitChunkKb k-blocks: the tensor core adds into its accumulator with round-toward-zero, an
    // error that grows with the number of additions times |accumulator|, so the long sum is
    // formed by the epilogue warps in registers (round-to-nearest) from short in-core sums.
    if (lane == 0) {
      // Descriptors are built once (address 0) and advanced with 64-bit adds: the start-address
      // field counts 16-byte units, so a stage offset or a k-step is one addition. Keeping the
      // per-MMA instruction count minimal matters: a single thread issues the MMAs, and with
      // descriptor construction inside the loop its instruction latency (~140 clk per MMA), not the
      // tensor core (128 clk per N=256 MMA), bounded the loop.
      constexpr uint32_t idesc = BF16 ? make_idesc_bf16(128, BN) : make_idesc(BN, B_MN);
      constexpr uint32_t kStage16 = C::kStageBytes >> 4;
      constexpr uint32_t kAStep = (UMMA_K * 4) >> 4;                         // 32 B inside the swizzle row
      constexpr uint32_t kBStep = B_MN ? (1024 >> 4) : ((UMMA_K * 4) >> 4);  // next 8 k-rows, or 32 B
      const uint64_t a_desc0 = make_smem_desc(smem_base, 16, 1024, kLayoutSw128);
      const uint64_t b_desc0 = B_MN ? make_smem_desc(smem_base + A_STAGE_BYTES, BK * 128, 512, kLayoutSw128Base32)
                                    : make_smem_desc(smem_base + A_STAGE_BYTES, 16, 1024, kLayoutSw128);
      constexpr uint32_t kBLo16 = C::kBStageBytes >> 4;  // B_hi -> B_lo of the same stage
      const int chunk = SPLIT3 ? kSplitChunkKb : p.num_kb;
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
        for (int kb0 = 0; kb0 < p.num_kb && ok; kb0 += chunk) {
          if (!(ok = mbar_wait(bar_tempty + 8 * acc, acc_ph ^ 1, abort_flag, p.status, 2u))) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
          const int kb_end = kb0 + chunk < p.num_kb ? kb0 + chunk : p.num_kb;
          for (int kb = kb0; kb < kb_end; ++kb) {
            if (!(ok = mbar_wait((SPLIT3 ? bar_split : bar_full) + 8 * s, ph, abort_flag, p.status, 4u))) break;
            tc_fence_after();
            const uint64_t a_hi = a_desc0 + (uint32_t)s * kStage16;
            const uint64_t b_hi = b_desc0 + (uint32_t)s * kStage16;
            const uint32_t first = kb > kb0 ? 1u : 0u;  // 0: the chunk's first MMA overwrites the accumulator
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk) {
              const uint32_t accumulate = kk > 0 ? 1u : first;
              if (SPLIT3) {
                // A operand from TMEM: 32 columns of hi then 32 of lo per stage, 8 columns per k-step
                const uint32_t a_hi_t = tmem_base + C::kASplitCol0 + (uint32_t)s * 64 + kk * UMMA_K;
                umma_tf32_ts(d_tmem, a_hi_t + 32, b_hi + kk * kBStep, idesc, accumulate);      // lo * hi
                umma_tf32_ts(d_tmem, a_hi_t, b_hi + kBLo16 + kk * kBStep, idesc, 1u);          // hi * lo
                umma_tf32_ts(d_tmem, a_hi_t, b_hi + kk * kBStep, idesc, 1u);                   // hi * hi
              } else if (BF16) {
                umma_bf16(d_tmem, a_hi + kk * kAStep, b_hi + kk * kBStep, idesc, accumulate);
              } else {
                umma_tf32(d_tmem, a_hi + kk * kAStep, b_hi + kk * kBStep, idesc, accumulate);
              }
            }
            umma_commit(bar_empty + 8 * s);  // stage reusable once these MMAs have read it
            if (++s == kStages) { s = 0; ph ^= 1; }
          }
          if (!ok) break;
          umma_commit(bar_tfull + 8 * acc);  // this chunk's accumulator is complete
          if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
      }
    }
  } else if (warp < 2 + C::kEpilogueWarps) {
    // ------------------------------- epilogue -------------------------------
    // Warp w reads TMEM lanes [32*(w%4), +32); the warps of a lane quarter split the columns.
    const int ew = warp - 2;
    const int quarter = warp & 3;
    const int col0 = (ew >> 2) * C::kColsPerWarp;
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    for (int64_t tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
      const int n_t = (int)(tile % p.num_n_tiles);
      const int64_t r = tile / p.num_n_tiles;
      const int m_t = (int)(r % p.num_m_tiles);
      const int64_t batch = r / p.num_m_tiles;
      const int64_t bo = batch / p.batch_inner, bi = batch % p.batch_inner;
      const int64_t m = (int64_t)m_t * BM + quarter * 32 + lane;
      const int64_t row_off = bo * p.y_stride_outer + bi * p.y_stride_inner + m * p.ldy;
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
      // convolution: this thread's row is one output pixel of one of the tile's two 8x8 blocks
      bool cv_valid = false;
      int64_t cv_off = 0, cv_cs = 0;
      if (CONV) {
        const int row = quarter * 32 + lane;
        const int64_t blk = 2 * (int64_t)m_t + (row >> 6);
        const int img = (int)(blk / p.cv.blocks_per_img);
        const int rem = (int)(blk - (int64_t)img * p.cv.blocks_per_img);
        const int by = rem / p.cv.blocks_w, bx = rem - by * p.cv.blocks_w;
        const int oh = by * 8 + ((row & 63) >> 3), ow = bx * 8 + (row & 7);
        cv_valid = blk < p.cv.total_blocks && oh < p.cv.OH && ow < p.cv.OW;
        cv_cs = (int64_t)p.cv.OH * p.cv.OW;
        cv_off = (int64_t)img * p.N * cv_cs + (int64_t)oh * p.cv.OW + ow;
      }
      auto finish_block = [&](float *v, int c0) {
        if (CONV) finish_pixel32(p, v, cv_valid, cv_off, cv_cs, (int64_t)n_t * BN + c0);
        else finish_row32(p, v, m, row_off, (int64_t)n_t * BN + c0);
      };
      if (SPLIT3) {
        // Sum the per-chunk accumulators in registers, then apply the epilogue once.
        float sum[C::kColsPerWarp];
#pragma unroll
        for (int j = 0; j < C::kColsPerWarp; ++j) sum[j] = 0.f;
        for (int kb0 = 0; kb0 < p.num_kb; kb0 += kSplitChunkKb) {
          if (!(ok = mbar_wait(bar_tfull + 8 * acc, acc_ph, abort_flag, p.status, 8u))) break;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < C::kColsPerWarp; c += 16) {  // 16 columns at a time: keeps registers for `sum`
            uint32_t v[16];
            tmem_ld16(lane_addr + (uint32_t)(acc * BN + col0 + c), v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) sum[c + j] += __uint_as_float(v[j]);
          }
          tc_fence_before();
          mbar_arrive(bar_tempty + 8 * acc);
          if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
        if (!ok) break;
#pragma unroll
        for (int c = 0; c < C::kColsPerWarp; c += 32) finish_block(&sum[c], col0 + c);
      } else {
        if (!(ok = mbar_wait(bar_tfull + 8 * acc, acc_ph, abort_flag, p.status, 8u))) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < C::kColsPerWarp; c += 32) {
          uint32_t v[32];
          float f[32];
          tmem_ld32(lane_addr + (uint32_t)(acc * BN + col0 + c), v);
          tmem_ld_wait();
          if (c + 32 >= C::kColsPerWarp) {
            // last read of this accumulator by this thread: hand it back before the stores
            tc_fence_before();
            mbar_arrive(bar_tempty + 8 * acc);
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
          finish_block(f, col0 + c);
        }
        if (++acc == 2) { acc = 0; acc_ph ^= 1; }
      }
    }
  } else if (SPLIT3) {
    // ------------------------------- 3xTF32 split warps -------------------------------
    // Each landed stage is split into hi = tf32(x) and lo = tf32(x - hi).
    //  * A: thread = row (the warp's TMEM lane quarter). The row's 32 values are read from the
    //    128B-swizzled tile (16-byte chunk c of row r sits at chunk c ^ (r % 8)) and the two halves
    //    are written to TMEM, where the MMAs read their A operand: A costs shared memory one read.
    //  * B: split elementwise in shared memory (hi in place, lo beside it); the swizzled placement
    //    of each chunk is preserved by writing at the same offset.
    // Shared-memory bandwidth bounds this mode (tile traffic + the MMAs' B reads), hence A in TMEM.
    const int t = threadIdx.x - 32 * C::kSplitWarp0;  // 0..255
    const int quarter = warp & 3;
    const int colhalf = (warp - C::kSplitWarp0) >> 2;  // which 16 of the row's 32 values this warp splits
    const int row = quarter * 32 + lane;
    const uint32_t a_lane = tmem_base + ((uint32_t)(quarter * 32) << 16) + C::kASplitCol0 + colhalf * 16;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int64_t tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
      for (int kb = 0; kb < p.num_kb; ++kb) {
        if (!(ok = mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 16u))) break;
        uint8_t *stage = smem + (size_t)s * C::kStageBytes;
        {
          const float4 *arow = reinterpret_cast<const float4 *>(stage + row * 128);
          uint32_t hi[16], lo[16];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float4 x = arow[(colhalf * 4 + c) ^ (row & 7)];
            const float h0 = to_tf32_rna(x.x), h1 = to_tf32_rna(x.y), h2 = to_tf32_rna(x.z), h3 = to_tf32_rna(x.w);
            hi[4 * c + 0] = __float_as_uint(h0); hi[4 * c + 1] = __float_as_uint(h1);
            hi[4 * c + 2] = __float_as_uint(h2); hi[4 * c + 3] = __float_as_uint(h3);
            lo[4 * c + 0] = __float_as_uint(to_tf32_rna(x.x - h0)); lo[4 * c + 1] = __float_as_uint(to_tf32_rna(x.y - h1));
            lo[4 * c + 2] = __float_as_uint(to_tf32_rna(x.z - h2)); lo[4 * c + 3] = __float_as_uint(to_tf32_rna(x.w - h3));
          }
          tmem_st16(a_lane + (uint32_t)s * 64, hi);
          tmem_st16(a_lane + (uint32_t)s * 64 + 32, lo);
        }
        float4 *src = reinterpret_cast<float4 *>(stage + A_STAGE_BYTES);
        float4 *dst_lo = reinterpret_cast<float4 *>(stage + A_STAGE_BYTES + C::kBStageBytes);
        constexpr int kVecs = C::kBStageBytes / 16;
#pragma unroll 4
        for (int i = t; i < kVecs; i += 32 * C::kSplitWarps) {
          const float4 x = src[i];
          float4 hi, lo;
          hi.x = to_tf32_rna(x.x); hi.y = to_tf32_rna(x.y); hi.z = to_tf32_rna(x.z); hi.w = to_tf32_rna(x.w);
          lo.x = to_tf32_rna(x.x - hi.x); lo.y = to_tf32_rna(x.y - hi.y);
          lo.z = to_tf32_rna(x.z - hi.z); lo.w = to_tf32_rna(x.w - hi.w);
          src[i] = hi;
          dst_lo[i] = lo;
        }
        // Publish: TMEM stores complete, generic-proxy shared-memory writes visible to the tensor core.
        tmem_st_wait();
        tc_fence_before();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(bar_split + 8 * s);
        if (++s == kStages) { s = 0; ph ^= 1; }
      }
    }
  }

  // Teardown: all roles meet, then the allocating warp returns the TMEM columns.
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (s_abort) {
    // Give loads that were already issued time to land before the CTA's shared memory is released.
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// CTA-pair variant (TF32 mode, dense GEMM): a cluster of two CTAs computes a 256 x BN tile.
// Each CTA loads its 128 rows of A and HALF of the B tile (BN/2 columns); the even CTA issues
// tcgen05.mma.cta_group::2 (M = 256), which reads B from both CTAs' shared memory and writes each
// CTA's 128 x BN accumulator into its own TMEM. Per FLOP this halves the B traffic from L2 into
// shared memory, the B operand reads of the tensor core and the number of MMA instructions, and
// leaves room for six pipeline stages. Roles per CTA are as in the single-CTA kernel; barriers:
//   full[s]    in the even CTA, 1 arrival (its expect_tx for both CTAs' bytes) + those bytes
//   empty[s]   in each CTA, 1 arrival: the even CTA commits to both
//   tfull[a]   in each CTA, 1 arrival: the even CTA commits to both
//   tempty[a]  in the even CTA, one arrival per epilogue thread of both CTAs
// ---------------------------------------------------------------------------------------------

template <int BN>
struct Cfg2 {
  static constexpr int kBHalfBytes = (BN / 2) * BK * 4;
  // Two k-blocks per pipeline stage: the issuing thread pays its barrier wait, commit and loop
  // overhead once per eight MMAs instead of once per four, which keeps it ahead of the tensor core.
  static constexpr int kKbPerStage = 2;
  static constexpr int kStageBytes = kKbPerStage * (A_STAGE_BYTES + kBHalfBytes);
  static constexpr int kStages = (192 * 1024) / kStageBytes > 8 ? 8 : (192 * 1024) / kStageBytes;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kWarpsPerQuarter = 4;
  static constexpr int kEpilogueWarps = 4 * kWarpsPerQuarter;
  static constexpr int kThreads = 32 * (2 + kEpilogueWarps);
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
  static constexpr int kColsPerWarp = BN / kWarpsPerQuarter;
};

template <int BN, bool B_MN, bool BF16 = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg2<BN>::kThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmParams p) {
  using C = Cfg2<BN>;
  constexpr int kStages = C::kStages;
  constexpr int BKE = BF16 ? 64 : BK;  // elements of K per k-block (one 128-byte row)
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kStages * C::kStageBytes);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * kStages;
  const uint32_t bar_tfull = bar_empty + 8 * kStages;
  const uint32_t bar_tempty = bar_tfull + 16;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t rank = cluster_ctarank();  // 0: issues the MMAs, 1: its partner
  const int64_t pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 2 * C::kEpilogueWarps);  // one arrival per epilogue warp of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&s_tmem_base), C::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before either touches the other's
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int *abort_flag = &s_abort;
  // p.num_m_tiles counts 256-row tile pairs here
  const int64_t num_tiles = (int64_t)p.num_m_tiles * p.num_n_tiles * (p.num_tiles_batch);

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) -------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      const uint32_t full_pair0 = map_to_cta(bar_full, 0);
      for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int n_t = (int)(tile % p.num_n_tiles);
        const int64_t r = tile / p.num_n_tiles;
        const int m_t = (int)(r % p.num_m_tiles);
        const int64_t batch = r / p.num_m_tiles;
        const int bo = (int)(batch / p.batch_inner), bi = (int)(batch % p.batch_inner);
        const int row0 = (2 * m_t + (int)rank) * BM;
        const int col0 = n_t * BN + (int)rank * (BN / 2);
        for (int kb = 0; kb < p.num_kb; kb += C::kKbPerStage) {
          if (!(ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 1u))) break;
          // One expect_tx per stage, posted locally by the even CTA for the bytes of BOTH CTAs; the
          // partner only issues its loads, whose completions are counted on the even CTA's barrier.
          // (Its bytes can only arrive after the stage's previous phase has completed, because its
          // own `empty` wait above is released by a commit that follows that completion.)
          // Stage layout: [A kb][A kb+1][B kb][B kb+1]; a k-block past the end of K is zero-filled.
          const uint32_t stage = smem_base + s * C::kStageBytes;
          const uint32_t full = rank == 0 ? bar_full + 8 * s : full_pair0 + 8 * s;
          if (rank == 0) mbar_expect_tx(bar_full + 8 * s, 2 * C::kStageBytes);
#pragma unroll
          for (int h = 0; h < C::kKbPerStage; ++h) {
            const uint32_t a_dst = stage + h * A_STAGE_BYTES;
            const uint32_t b_dst = stage + C::kKbPerStage * A_STAGE_BYTES + h * C::kBHalfBytes;
            const int k0 = (kb + h) * BKE;
            if (rank == 0) {
              tma_load_4d(a_dst, &map_a, full, k0, row0, bi * p.a_bi, bo * p.a_bo);
              if (B_MN) {
#pragma unroll
                for (int j = 0; j < BN / 64; ++j)
                  tma_load_4d(b_dst + j * (BK * 128), &map_b, full, col0 + 32 * j, k0, bi * p.b_bi, bo * p.b_bo);
              } else {
                tma_load_4d(b_dst, &map_b, full, k0, col0, bi * p.b_bi, bo * p.b_bo);
              }
            } else {
              tma_load_4d_pair(a_dst, &map_a, full, k0, row0, bi * p.a_bi, bo * p.a_bo);
              if (B_MN) {
#pragma unroll
                for (int j = 0; j < BN / 64; ++j)
                  tma_load_4d_pair(b_dst + j * (BK * 128), &map_b, full, col0 + 32 * j, k0, bi * p.b_bi, bo * p.b_bo);
              } else {
                tma_load_4d_pair(b_dst, &map_b, full, k0, col0, bi * p.b_bi, bo * p.b_bo);
              }
            }
          }
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (even CTA only) -------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = BF16 ? make_idesc_bf16(256, BN) : make_idesc_pair(BN, B_MN);
      constexpr uint32_t kStage16 = C::kStageBytes >> 4;
      constexpr uint32_t kAStep = (UMMA_K * 4) >> 4;
      constexpr uint32_t kBStep = B_MN ? (1024 >> 4) : ((UMMA_K * 4) >> 4);
      constexpr uint32_t kBOff = C::kKbPerStage * A_STAGE_BYTES;
      const uint64_t a_desc0 = make_smem_desc(smem_base, 16, 1024, kLayoutSw128);
      const uint64_t b_desc0 = B_MN ? make_smem_desc(smem_base + kBOff, BK * 128, 512, kLayoutSw128Base32)
                                    : make_smem_desc(smem_base + kBOff, 16, 1024, kLayoutSw128);
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        if (!(ok = mbar_wait(bar_tempty + 8 * acc, acc_ph ^ 1, abort_flag, p.status, 2u))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < p.num_kb; kb += C::kKbPerStage) {
          if (!(ok = mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 4u))) break;
          tc_fence_after();
          const uint64_t a_d = a_desc0 + (uint32_t)s * kStage16, b_d = b_desc0 + (uint32_t)s * kStage16;
          const uint32_t first = kb > 0 ? 1u : 0u;
#pragma unroll
          for (int h = 0; h < C::kKbPerStage; ++h) {
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk) {
              if (BF16)
                umma_bf16_pair(d_tmem, a_d + h * (A_STAGE_BYTES >> 4) + kk * kAStep,
                               b_d + h * (C::kBHalfBytes >> 4) + kk * kBStep, idesc, (h > 0 || kk > 0) ? 1u : first);
              else
                umma_tf32_pair(d_tmem, a_d + h * (A_STAGE_BYTES >> 4) + kk * kAStep,
                               b_d + h * (C::kBHalfBytes >> 4) + kk * kBStep, idesc, (h > 0 || kk > 0) ? 1u : first);
            }
          }
          // the stage is reusable in both CTAs once these MMAs have read it
          umma_commit_pair_both(bar_empty + 8 * s, 3);
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair_both(bar_tfull + 8 * acc, 3);
        if (++acc == 2) { acc = 0; acc_ph ^= 1; }
      }
    }
  } else {
    // ------------------------------- epilogue (both CTAs, own 128 rows) -------------------------------
    const int ew = warp - 2;
    const int quarter = warp & 3;
    const int col0 = (ew >> 2) * C::kColsPerWarp;
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      const int n_t = (int)(tile % p.num_n_tiles);
      const int64_t r = tile / p.num_n_tiles;
      const int m_t = (int)(r % p.num_m_tiles);
      const int64_t batch = r / p.num_m_tiles;
      const int64_t bo = batch / p.batch_inner, bi = batch % p.batch_inner;
      const int64_t m = (int64_t)(2 * m_t + (int)rank) * BM + quarter * 32 + lane;
      const int64_t row_off = bo * p.y_stride_outer + bi * p.y_stride_inner + m * p.ldy;
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
      if (!(ok = mbar_wait(bar_tfull + 8 * acc, acc_ph, abort_flag, p.status, 8u))) break;
      tc_fence_after();
      const uint32_t tempty_pair = map_to_cta(bar_tempty + 8 * acc, 0);
#pragma unroll 1
      for (int c = 0; c < C::kColsPerWarp; c += 32) {
        uint32_t v[32];
        float f[32];
        tmem_ld32(lane_addr + (uint32_t)(acc * BN + col0 + c), v);
        tmem_ld_wait();
        if (c + 32 >= C::kColsPerWarp) {
          // this warp is done with the accumulator: one (possibly remote) arrival per warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(tempty_pair);
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
        finish_row32(p, f, m, row_off, (int64_t)n_t * BN + col0 + c);
      }
      if (++acc == 2) { acc = 0; acc_ph ^= 1; }
    }
  }

  // Teardown: neither CTA may leave while its partner can still signal its barriers or read its
  // shared memory through the pair's MMAs.
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (s_abort) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, C::kTmemCols);
  }
}


// ---------------------------------------------------------------------------------------------
// CTA-pair variant of the 3xTF32 mode: a cluster of two CTAs computes a 256 x 128 tile with
// tcgen05.mma.cta_group::2. B arrives already split (hi = tf32(B), lo = tf32(B - hi), written once per
// call into the caller's workspace by split_tf32_kernel), so each CTA loads its 128 rows of raw A and
// 64 of the 128 tile columns of B_hi and B_lo; its split warps only turn A into hi / lo halves in TMEM.
// Per FLOP this halves the B operand reads of the tensor core and removes the B split from shared
// memory, whose bandwidth bounds the single-CTA 3xTF32 kernel. Chunked accumulation as there: every
// kSplitChunkKb k-blocks go to their own TMEM buffer and the epilogue warps sum the chunks in registers.
// Barriers (same offsets in both CTAs):
//   full[s]    own CTA: its TMA bytes of stage s            empty[s]  own CTA: multicast commit of the issuer
//   split[s]   even CTA: one arrival per split warp of both CTAs (A halves of stage s are in TMEM)
//   tfull[a]   own CTA: multicast commit                    tempty[a] even CTA: one arrival per epilogue warp of both
// ---------------------------------------------------------------------------------------------
// BN_ = 128 or 192 tile columns. One thread issues every MMA at ~68 clk per instruction, which for N = 128
// (64 clk of tensor work on the pair) leaves the tensor cores waiting; N = 192 instructions (96 clk) hide it.
template <int BN_>
struct Cfg3P {
  static constexpr int BN = BN_;
  static constexpr int kBHalfBytes = (BN / 2) * BK * 4;                  // half the tile columns of one B half
  static constexpr int kStageBytes = A_STAGE_BYTES + 2 * kBHalfBytes;    // A raw | B_hi | B_lo
  static constexpr int kStages = (200 * 1024) / kStageBytes > 6 ? 6 : (200 * 1024) / kStageBytes;  // TMA run-ahead
  static constexpr int kSlots = (512 - 2 * BN) / 64;                     // A hi/lo slots in TMEM (64 columns each)
  static constexpr int kASplitCol0 = 2 * BN;
  static constexpr int kTmemCols = 512;
  static constexpr int kColsPerWarp = 64;
  static constexpr int kEpilogueWarps = 4 * (BN / kColsPerWarp), kSplitWarps = 8;
  static constexpr int kSplitWarp0 = 2 + kEpilogueWarps;
  static constexpr int kThreads = 32 * (2 + kEpilogueWarps + kSplitWarps);
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256 + kEpilogueWarps * kColsPerWarp * 4;  // + barriers + staged bias
};

template <int BN_, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg3P<BN_>::kThreads, 1)
gemm_tc_pair3_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_bh,
                     const __grid_constant__ CUtensorMap map_bl, const GemmParams p) {
  using C = Cfg3P<BN_>;
  constexpr int kStages = C::kStages;
  constexpr int BN = C::BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kStages * C::kStageBytes);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * kStages;
  const uint32_t bar_split = bar_empty + 8 * kStages;  // one per TMEM slot
  const uint32_t bar_tfull = bar_split + 8 * C::kSlots;
  const uint32_t bar_tempty = bar_tfull + 16;
  float *bias_all = reinterpret_cast<float *>(smem + kStages * C::kStageBytes + 256);  // 64 bias values per epilogue warp
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t rank = cluster_ctarank();
  const int64_t pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int t = 0; t < C::kSlots; ++t) mbar_init(bar_split + 8 * t, 2 * C::kSplitWarps);
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 2 * C::kEpilogueWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&s_tmem_base), C::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int *abort_flag = &s_abort;
  const int64_t num_tiles = (int64_t)p.num_m_tiles * p.num_n_tiles;  // p.num_m_tiles counts 256-row pairs

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs, own barrier) -------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int n_t = (int)(tile % p.num_n_tiles);
        const int m_t = (int)(tile / p.num_n_tiles);
        const int row0 = (2 * m_t + (int)rank) * BM;
        const int col0 = n_t * BN + (int)rank * (BN / 2);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!(ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 1u))) break;
          const uint32_t stage = smem_base + s * C::kStageBytes;
          const uint32_t full = bar_full + 8 * s;
          mbar_expect_tx(full, C::kStageBytes);
          tma_load_4d(stage, &map_a, full, kb * BK, row0, 0, 0);
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) {
              tma_load_4d(stage + A_STAGE_BYTES + j * (BK * 128), &map_bh, full, col0 + 32 * j, kb * BK, 0, 0);
              tma_load_4d(stage + A_STAGE_BYTES + C::kBHalfBytes + j * (BK * 128), &map_bl, full, col0 + 32 * j,
                          kb * BK, 0, 0);
            }
          } else {
            tma_load_4d(stage + A_STAGE_BYTES, &map_bh, full, kb * BK, col0, 0, 0);
            tma_load_4d(stage + A_STAGE_BYTES + C::kBHalfBytes, &map_bl, full, kb * BK, col0, 0, 0);
          }
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (even CTA only) -------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_pair(BN, B_MN);
      constexpr uint32_t kStage16 = C::kStageBytes >> 4;
      constexpr uint32_t kBStep = B_MN ? (1024 >> 4) : ((UMMA_K * 4) >> 4);
      constexpr uint32_t kBLo16 = C::kBHalfBytes >> 4;
      const uint64_t b_desc0 = B_MN ? make_smem_desc(smem_base + A_STAGE_BYTES, BK * 128, 512, kLayoutSw128Base32)
                                    : make_smem_desc(smem_base + A_STAGE_BYTES, 16, 1024, kLayoutSw128);
      int s = 0, slot = 0;
      uint32_t slot_ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        for (int kb0 = 0; kb0 < p.num_kb && ok; kb0 += kSplitChunkKb) {
          if (!(ok = mbar_wait(bar_tempty + 8 * acc, acc_ph ^ 1, abort_flag, p.status, 2u))) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
          const int kb_end = kb0 + kSplitChunkKb < p.num_kb ? kb0 + kSplitChunkKb : p.num_kb;
          for (int kb = kb0; kb < kb_end; ++kb) {
            // both CTAs' split warps have put this k-block's A halves into TMEM slot `slot` (which also
            // means both CTAs' loads of shared-memory stage s have landed)
            if (!(ok = mbar_wait(bar_split + 8 * slot, slot_ph, abort_flag, p.status, 4u))) break;
            tc_fence_after();
            const uint64_t b_hi = b_desc0 + (uint32_t)s * kStage16;
            const uint32_t first = kb > kb0 ? 1u : 0u;
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk) {
              const uint32_t a_hi_t = tmem_base + C::kASplitCol0 + (uint32_t)slot * 64 + kk * UMMA_K;
              umma_tf32_ts_pair(d_tmem, a_hi_t + 32, b_hi + kk * kBStep, idesc, kk > 0 ? 1u : first);  // lo * hi
              umma_tf32_ts_pair(d_tmem, a_hi_t, b_hi + kBLo16 + kk * kBStep, idesc, 1u);                // hi * lo
              umma_tf32_ts_pair(d_tmem, a_hi_t, b_hi + kk * kBStep, idesc, 1u);                         // hi * hi
            }
            umma_commit_pair_both(bar_empty + 8 * s, 3);
            if (++s == kStages) s = 0;
            if (++slot == C::kSlots) { slot = 0; slot_ph ^= 1; }
          }
          if (!ok) break;
          umma_commit_pair_both(bar_tfull + 8 * acc, 3);
          if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
      }
    }
  } else if (warp < C::kSplitWarp0) {
    // ------------------------------- epilogue (both CTAs, own 128 rows) -------------------------------
    const int ew = warp - 2;
    const int quarter = warp & 3;
    const int col0 = (ew >> 2) * C::kColsPerWarp;
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      const int n_t = (int)(tile % p.num_n_tiles);
      const int m_t = (int)(tile / p.num_n_tiles);
      const int64_t m = (int64_t)(2 * m_t + (int)rank) * BM + quarter * 32 + lane;
      const int64_t row_off = m * p.ldy;
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
      // Stage this warp's 64 bias values in its own shared-memory slice while the tile's first chunk is
      // still being computed: the store phase then reads them as broadcast 128-bit loads.
      float *bias_s = bias_all + ew * C::kColsPerWarp;
      if (p.bias) {
        const int64_t n = (int64_t)n_t * BN + col0 + lane;
        bias_s[lane] = n < p.N ? __ldg(p.bias + n) : 0.f;
        bias_s[32 + lane] = n + 32 < p.N ? __ldg(p.bias + n + 32) : 0.f;
      }
      __syncwarp();
      float sum[C::kColsPerWarp];
#pragma unroll
      for (int j = 0; j < C::kColsPerWarp; ++j) sum[j] = 0.f;
      for (int kb0 = 0; kb0 < p.num_kb; kb0 += kSplitChunkKb) {
        if (!(ok = mbar_wait(bar_tfull + 8 * acc, acc_ph, abort_flag, p.status, 8u))) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < C::kColsPerWarp; c += 16) {
          uint32_t v[16];
          tmem_ld16(lane_addr + (uint32_t)(acc * BN + col0 + c), v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) sum[c + j] += __uint_as_float(v[j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (rank == 0) mbar_arrive(bar_tempty + 8 * acc);
          else mbar_arrive_cluster_relaxed(map_to_cta(bar_tempty + 8 * acc, 0));
        }
        if (++acc == 2) { acc = 0; acc_ph ^= 1; }
      }
      if (!ok) break;
#pragma unroll
      for (int c = 0; c < C::kColsPerWarp; c += 32)
        finish_row32(p, &sum[c], m, row_off, (int64_t)n_t * BN + col0 + c, p.bias ? bias_s + c : nullptr);
      __syncwarp();  // all lanes have read the staged bias before the next tile's values replace it
    }
  } else {
    // ------------------------------- split warps: A -> hi / lo halves in TMEM -------------------------------
    const int quarter = warp & 3;
    const int colhalf = (warp - C::kSplitWarp0) >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t a_lane = tmem_base + ((uint32_t)(quarter * 32) << 16) + C::kASplitCol0 + colhalf * 16;
    const uint32_t split_pair0 = map_to_cta(bar_split, 0);
    int s = 0, slot = 0;
    uint32_t ph = 0;
    // The slot was last read by the MMAs of the k-block kSlots before this one; they release shared-memory
    // stage `rs` (the stage that k-block used) through empty[rs], whose phase `rph` this thread tracks.
    int rs = 0;
    uint32_t rph = 0;
    int64_t n = 0;  // k-blocks processed so far by this CTA
    bool ok = true;
    for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      for (int kb = 0; kb < p.num_kb; ++kb, ++n) {
        if (n >= C::kSlots) {
          if (!(ok = mbar_wait(bar_empty + 8 * rs, rph, abort_flag, p.status, 32u))) break;
          if (++rs == kStages) { rs = 0; rph ^= 1; }
        }
        if (!(ok = mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 16u))) break;
        const float4 *arow = reinterpret_cast<const float4 *>(smem + (size_t)s * C::kStageBytes + row * 128);
        uint32_t hi[16], lo[16];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float4 x = arow[(colhalf * 4 + c) ^ (row & 7)];
          const float h0 = to_tf32_rna(x.x), h1 = to_tf32_rna(x.y), h2 = to_tf32_rna(x.z), h3 = to_tf32_rna(x.w);
          hi[4 * c + 0] = __float_as_uint(h0); hi[4 * c + 1] = __float_as_uint(h1);
          hi[4 * c + 2] = __float_as_uint(h2); hi[4 * c + 3] = __float_as_uint(h3);
          lo[4 * c + 0] = __float_as_uint(to_tf32_rna(x.x - h0)); lo[4 * c + 1] = __float_as_uint(to_tf32_rna(x.y - h1));
          lo[4 * c + 2] = __float_as_uint(to_tf32_rna(x.z - h2)); lo[4 * c + 3] = __float_as_uint(to_tf32_rna(x.w - h3));
        }
        tc_fence_after();
        tmem_st16(a_lane + (uint32_t)slot * 64, hi);
        tmem_st16(a_lane + (uint32_t)slot * 64 + 32, lo);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          // the even CTA's own barrier takes a plain arrival; the partner's crosses the cluster without a release
          if (rank == 0) mbar_arrive(bar_split + 8 * slot);
          else mbar_arrive_cluster_relaxed(split_pair0 + 8 * slot);
        }
        if (++s == kStages) { s = 0; ph ^= 1; }
        if (++slot == C::kSlots) slot = 0;
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (s_abort) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, C::kTmemCols);
  }
}

// hi = tf32(x), lo = tf32(x - hi) of a [rows, cols] matrix with row pitch ld, written densely (pitch ldp)
__global__ void __launch_bounds__(256)
split_tf32_kernel(const float *__restrict__ x, float *__restrict__ hi, float *__restrict__ lo, int64_t rows, int64_t cols4,
                  int64_t ld, int64_t ldp) {
  const int64_t total = rows * cols4;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / cols4, c = (i - r * cols4) * 4;
    const float4 v = *reinterpret_cast<const float4 *>(x + r * ld + c);
    float4 h, l;
    h.x = to_tf32_rna(v.x); h.y = to_tf32_rna(v.y); h.z = to_tf32_rna(v.z); h.w = to_tf32_rna(v.w);
    l.x = to_tf32_rna(v.x - h.x); l.y = to_tf32_rna(v.y - h.y); l.z = to_tf32_rna(v.z - h.z); l.w = to_tf32_rna(v.w - h.w);
    *reinterpret_cast<float4 *>(hi + r * ldp + c) = h;
    *reinterpret_cast<float4 *>(lo + r * ldp + c) = l;
  }
}

// ---------------------------------------------------------------------------------------------
// Host side: tensor-map encoding and launch
// ---------------------------------------------------------------------------------------------
// A batch axis that is broadcast (stride 0) or trivial (extent 1) is encoded with extent 1 and a
// valid dummy stride; the kernel then always passes coordinate 0 on it.
void batch_axis(int64_t extent, int64_t stride_elems, uint64_t fallback_bytes, uint64_t *dim, uint64_t *stride_bytes,
                int *advances) {
  if (extent > 1 && stride_elems != 0) {
    *dim = (uint64_t)extent;
    *stride_bytes = (uint64_t)stride_elems * 4;
    *advances = 1;
  } else {
    *dim = 1;
    *stride_bytes = fallback_bytes;
    *advances = 0;
  }
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) is per (function, device) and sticks: do it once each.
// `done` is the caller's per-kernel flag word (bit d: set on device d).
template <typename Kernel>
int raise_dynamic_smem_once(Kernel kern, int bytes, const char *what, std::atomic<uint64_t> &done) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(B200_ECUDA, "%s: bad device", what);
  if (done.load(std::memory_order_relaxed) >> dev & 1) return B200_OK;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
    return fail(B200_ECUDA, "%s: cannot set dynamic shared memory to %d", what, bytes);
  done.fetch_or(1ull << dev, std::memory_order_relaxed);
  return B200_OK;
}

template <int BN, bool B_MN, bool SPLIT3, bool CONV = false, bool BF16 = false>
int launch_cfg(cudaStream_t st, const CUtensorMap &ma, const CUtensorMap &mb, GemmParams &p) {
  using C = Cfg<BN, SPLIT3>;
  auto kern = gemm_tc_kernel<BN, B_MN, SPLIT3, CONV, BF16>;
  static std::atomic<uint64_t> smem_set{0};  // one per kernel instantiation
  if (int rc = raise_dynamic_smem_once(kern, C::kSmemBytes, "gemm(tc)", smem_set)) return rc;
  const int64_t grid = p.num_tiles < kNumSMs ? p.num_tiles : kNumSMs;
  kern<<<(unsigned)grid, C::kThreads, C::kSmemBytes, st>>>(ma, mb, p);
  return check_launch("gemm_tc");
}

template <int BN, bool B_MN, bool BF16 = false>
int launch_pair(cudaStream_t st, const CUtensorMap &ma, const CUtensorMap &mb, GemmParams &p) {
  using C = Cfg2<BN>;
  auto kern = gemm_tc_pair_kernel<BN, B_MN, BF16>;
  static std::atomic<uint64_t> smem_set{0};  // one per kernel instantiation
  if (int rc = raise_dynamic_smem_once(kern, C::kSmemBytes, "gemm(tc pair)", smem_set)) return rc;
  // A persistent grid must not exceed the clusters the device can hold at once (both CTAs of a
  // pair sit in one GPC, so this is fewer than SMs / 2); extra clusters would run a second wave alone.
  static std::atomic<int> max_pairs[64];  // per device (zero-initialised); depends only on the kernel and its resources
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(B200_ECUDA, "gemm(tc pair): bad device");
  if (max_pairs[dev].load(std::memory_order_relaxed) == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kNumSMs, 1, 1);
    cfg.blockDim = dim3(C::kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1)
      return fail(B200_ECUDA, "gemm(tc pair): cudaOccupancyMaxActiveClusters failed");
    max_pairs[dev].store(n, std::memory_order_relaxed);
  }
  const int64_t tiles = (int64_t)p.num_m_tiles * p.num_n_tiles * p.num_tiles_batch;
  const int64_t cap = max_pairs[dev].load(std::memory_order_relaxed);
  const int64_t pairs = tiles < cap ? tiles : cap;
  kern<<<(unsigned)(2 * pairs), C::kThreads, C::kSmemBytes, st>>>(ma, mb, p);
  return check_launch("gemm_tc_pair");
}

template <int BN, bool B_MN>
int launch_pair3(cudaStream_t st, const CUtensorMap &ma, const CUtensorMap &mbh, const CUtensorMap &mbl, GemmParams &p) {
  using C = Cfg3P<BN>;
  auto kern = gemm_tc_pair3_kernel<BN, B_MN>;
  static std::atomic<uint64_t> smem_set{0};  // one per kernel instantiation
  if (int rc = raise_dynamic_smem_once(kern, C::kSmemBytes, "gemm(tc pair3)", smem_set)) return rc;
  static std::atomic<int> max_pairs[64];  // per device, as in launch_pair
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(B200_ECUDA, "gemm(tc pair3): bad device");
  if (max_pairs[dev].load(std::memory_order_relaxed) == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kNumSMs, 1, 1);
    cfg.blockDim = dim3(C::kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1)
      return fail(B200_ECUDA, "gemm(tc pair3): cudaOccupancyMaxActiveClusters failed");
    max_pairs[dev].store(n, std::memory_order_relaxed);
  }
  const int64_t tiles = (int64_t)p.num_m_tiles * p.num_n_tiles;
  const int64_t cap = max_pairs[dev].load(std::memory_order_relaxed);
  const int64_t pairs = tiles < cap ? tiles : cap;
  kern<<<(unsigned)(2 * pairs), C::kThreads, C::kSmemBytes, st>>>(ma, mbh, mbl, p);
  return check_launch("gemm_tc_pair3");
}

template <bool B_MN, bool SPLIT3>
int launch_bn(cudaStream_t st, int bn, const CUtensorMap &ma, const CUtensorMap &mb, GemmParams &p) {
  switch (bn) {
    case 64: return launch_cfg<64, B_MN, SPLIT3>(st, ma, mb, p);
    case 128: return launch_cfg<128, B_MN, SPLIT3>(st, ma, mb, p);
    case 256:
      if constexpr (!SPLIT3) return launch_cfg<256, B_MN, false>(st, ma, mb, p);
  }
  return fail(B200_EINVAL, "gemm(tc): no kernel for BN=%d", bn);
}

template <bool SPLIT3>
int launch_conv_bn(cudaStream_t st, int bn, const CUtensorMap &ma, const CUtensorMap &mb, GemmParams &p) {
  switch (bn) {
    case 64: return launch_cfg<64, false, SPLIT3, true>(st, ma, mb, p);
    case 128: return launch_cfg<128, false, SPLIT3, true>(st, ma, mb, p);
    case 256:
      if constexpr (!SPLIT3) return launch_cfg<256, false, false, true>(st, ma, mb, p);
  }
  return fail(B200_EINVAL, "conv(tc): no kernel for BN=%d", bn);
}

inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

// fp32 [rows, cols] (row pitch ld) -> bf16 [rows, colsp], round-to-nearest-even, columns past `cols` zero; eight
// outputs (one 16-byte store) per thread. colsp is a multiple of 8.
__global__ void __launch_bounds__(256)
convert_bf16_kernel(const float *__restrict__ x, __nv_bfloat16 *__restrict__ out, int64_t rows, int64_t cols, int64_t ld,
                    int64_t colsp) {
  const int64_t per_row = colsp >> 3, total = rows * per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / per_row, c = (i - r * per_row) << 3;
    const float *src = x + r * ld + c;
    float v[8];
    if (c + 8 <= cols && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
      const float4 a = ld_stream4(src), b = ld_stream4(src + 4);
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = c + j < cols ? src[j] : 0.f;
    }
    __nv_bfloat162 q[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
    *reinterpret_cast<uint4 *>(out + r * colsp + c) = *reinterpret_cast<const uint4 *>(q);
  }
}

// fp32 [rows, cols] (row pitch ld) -> bf16 [cols, rowsp]: the transpose, so that a [K, N] operand becomes K-major
__global__ void __launch_bounds__(256)
convert_bf16_transpose_kernel(const float *__restrict__ x, __nv_bfloat16 *__restrict__ out, int64_t rows, int64_t cols,
                              int64_t ld, int64_t rowsp) {
  __shared__ float tile[32][33];
  const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int k = ty; k < 32; k += 8) tile[k][tx] = (r0 + k < rows && c0 + tx < cols) ? x[(r0 + k) * ld + c0 + tx] : 0.f;
  __syncthreads();
  for (int k = ty; k < 32; k += 8)
    if (c0 + k < cols && r0 + tx < rowsp) out[(c0 + k) * rowsp + r0 + tx] = __float2bfloat16_rn(tile[tx][k]);
}

int pick_bn(int64_t N, bool split3) {
  const int cands[3] = {256, 128, 64};
  int best = 64;
  double best_cost = 1e30;
  for (int i = split3 ? 1 : 0; i < 3; ++i) {
    const int bn = cands[i];
    const int64_t tiles = (N + bn - 1) / bn;
    // padded work, with a mild preference for wide tiles (fewer A re-reads, better MMA efficiency)
    const double cost = (double)(tiles * bn) * (bn == 256 ? 1.0 : bn == 128 ? 1.04 : 1.15);
    if (cost < best_cost) { best_cost = cost; best = bn; }
  }
  return best;
}

}  // namespace

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static std::atomic<EncodeTiledFn> cached{nullptr};  // process-wide driver entry point; identical for every device
  EncodeTiledFn fn = cached.load(std::memory_order_relaxed);
  if (!fn) {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
    cached.store(fn, std::memory_order_relaxed);
  }
  return fn;
}

// A caller with static shapes (a DaCe tasklet, a planned ONNX graph, a CUDA-graph capture) asks for the same
// tensor maps on every call. Each host thread keeps the last maps it encoded in a small direct-mapped table keyed by
// everything the encoding depends on (base address, extents, strides, box, swizzle); a hit is a 128-byte copy
// instead of a driver call. The table holds descriptors, never device memory.
namespace {
struct MapKey {
  const void *base;
  uint64_t dims[4], strides[3];
  uint32_t box[3], swizzle;
  bool operator==(const MapKey &o) const { return memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapSlot {
  bool valid = false;
  MapKey key;
  CUtensorMap map;
};
constexpr int kMapSlots = 64;
}  // namespace

int tc::encode_map(CUtensorMap *map, const float *base, const uint64_t dims[4], const uint64_t strides_bytes[3],
               uint32_t box0, uint32_t box1, CUtensorMapSwizzle swizzle, uint32_t box2) {
  static thread_local MapSlot table[kMapSlots];
  MapKey key;
  memset(&key, 0, sizeof(key));
  key.base = base;
  for (int i = 0; i < 4; ++i) key.dims[i] = dims[i];
  for (int i = 0; i < 3; ++i) key.strides[i] = strides_bytes[i];
  key.box[0] = box0; key.box[1] = box1; key.box[2] = box2;
  key.swizzle = (uint32_t)swizzle;
  uint64_t h = reinterpret_cast<uintptr_t>(base) * 0x9E3779B97F4A7C15ull;
  h ^= (dims[0] * 31 + dims[1]) * 0xC2B2AE3D27D4EB4Full + strides_bytes[0] * 131 + box0 * 7 + box1 * 3 + box2 + (uint64_t)swizzle;
  MapSlot &slot = table[(h >> 20) % kMapSlots];
  if (slot.valid && slot.key == key) {
    *map = slot.map;
    return B200_OK;
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return fail(B200_ECUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t gdim[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t gstr[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
  cuuint32_t box[4] = {box0, box1, box2, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(base), gdim, gstr, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(B200_ECUDA,
                "cuTensorMapEncodeTiled failed (%d): dims {%llu,%llu,%llu,%llu} strides {%llu,%llu,%llu} box {%u,%u}",
                (int)r, (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2],
                (unsigned long long)dims[3], (unsigned long long)strides_bytes[0],
                (unsigned long long)strides_bytes[1], (unsigned long long)strides_bytes[2], box0, box1);
  slot.valid = true;
  slot.key = key;
  slot.map = *map;
  return B200_OK;
}


int tc::encode_map_bf16(CUtensorMap *map, const void *base, uint64_t k, uint64_t rows, uint64_t pitch_bytes,
                        uint32_t box_k, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return fail(B200_ECUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t gdim[4] = {k, rows, 1, 1};
  cuuint64_t gstr[3] = {pitch_bytes, pitch_bytes * rows, pitch_bytes * rows};
  cuuint32_t box[4] = {box_k, box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), gdim, gstr, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(B200_ECUDA, "cuTensorMapEncodeTiled (bf16) failed (%d): k %llu rows %llu pitch %llu box {%u,%u}", (int)r,
                (unsigned long long)k, (unsigned long long)rows, (unsigned long long)pitch_bytes, box_k, box_rows);
  return B200_OK;
}

int tc::encode_map5(CUtensorMap *map, const float *base, const uint64_t dims[5], const uint64_t strides_bytes[4],
                    const uint32_t box[5], CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return fail(B200_ECUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t gdim[5] = {dims[0], dims[1], dims[2], dims[3], dims[4]};
  cuuint64_t gstr[4] = {strides_bytes[0], strides_bytes[1], strides_bytes[2], strides_bytes[3]};
  cuuint32_t bx[5] = {box[0], box[1], box[2], box[3], box[4]};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float *>(base), gdim, gstr, bx, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(B200_ECUDA, "cuTensorMapEncodeTiled (rank 5) failed (%d): dims {%llu,%llu,%llu,%llu,%llu} box {%u,%u,%u,%u,%u}",
                (int)r, (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2],
                (unsigned long long)dims[3], (unsigned long long)dims[4], box[0], box[1], box[2], box[3], box[4]);
  return B200_OK;
}


bool gemm_tc_supported(const b200_gemm_desc &d, const float *A, const float *B, const float *Y) {
  auto ok4 = [](int64_t v) { return v % 4 == 0; };
  if (d.M < 1 || d.N < 1 || d.K < 1) return false;
  if (!aligned16(A) || !aligned16(B)) return false;
  if (!ok4(d.lda) || !ok4(d.ldb)) return false;
  if (!ok4(d.a_stride_outer) || !ok4(d.a_stride_inner) || !ok4(d.b_stride_outer) || !ok4(d.b_stride_inner))
    return false;
  if (d.lda < d.K) return false;
  if (d.trans_b ? d.ldb < d.K : d.ldb < d.N) return false;
  if (d.M > 0x7fffffffLL || d.N > 0x7fffffffLL || d.K > 0x7fffffffLL) return false;
  if (d.batch_outer > 0x7fffffffLL || d.batch_inner > 0x7fffffffLL) return false;
  (void)Y;
  return true;
}

// 3xTF32 with a workspace: B is split once into dense hi / lo copies (row pitch = columns rounded up to 4)
// and the CTA-pair kernel runs. Qualifies: one matrix (no batch), more than one row tile, B rows a multiple of
// four floats long.
static bool pair3_qualifies(const b200_gemm_desc &d) {
  const int64_t cols = d.trans_b ? d.K : d.N;
  return d.math_mode == B200_MATH_FP32X3 && d.batch_outer * d.batch_inner == 1 && d.M > BM && cols % 4 == 0;
}
static size_t pair3_workspace_bytes(const b200_gemm_desc &d) {
  const int64_t rows = d.trans_b ? d.N : d.K, cols = d.trans_b ? d.K : d.N;
  return 2 * align256((size_t)rows * (size_t)cols * 4);
}
// Below ~9 GFLOP the extra launch of the split kernel and the pair kernel's longer prologue cost more than its
// faster main loop saves (measured: [4096,120] x 784 33 -> 29 us, [4096,84] x 120 19 -> 13 us on the plain path;
// [8192,768] x 768 66 -> 56 us with the workspace): such calls are told to bring no workspace.
static bool pair3_worth_it(const b200_gemm_desc &d) { return (double)d.M * (double)d.N * (double)d.K >= 4.5e9; }

// BF16 mode: one matrix (no batch). Both operands are converted into the workspace, K padded to a multiple of 8.
static bool bf16_qualifies(const b200_gemm_desc &d) {
  return d.math_mode == B200_MATH_BF16 && d.batch_outer * d.batch_inner == 1;
}
static size_t bf16_operand_bytes(int64_t rows, int64_t K) { return align256((size_t)rows * (size_t)((K + 7) / 8 * 8) * 2); }

size_t gemm_tc_workspace_bytes(const b200_gemm_desc &d) {
  if (bf16_qualifies(d)) return bf16_operand_bytes(d.M, d.K) + bf16_operand_bytes(d.N, d.K);
  if (!pair3_qualifies(d) || !pair3_worth_it(d)) return 0;
  return pair3_workspace_bytes(d);
}

// BF16 mode: A and B are rounded to bf16 into the workspace (B transposed to [N, K] when it is given as [K, N]), then
// the same tile kernels run with kind::f16 MMAs (K = 16 per instruction, twice the TF32 rate), fp32 accumulate.
static int gemm_tc_bf16(cudaStream_t st, const b200_gemm_desc &d, const float *A, const float *B, const float *bias,
                        const float *residual, float *Y, void *workspace, size_t workspace_bytes) {
  const size_t a_bytes = bf16_operand_bytes(d.M, d.K), b_bytes = bf16_operand_bytes(d.N, d.K);
  if (!workspace || workspace_bytes < a_bytes + b_bytes)
    return fail(B200_EWORKSPACE, "gemm(bf16): the BF16 mode converts its operands into a workspace of %zu bytes "
                                 "(b200_gemm_workspace_bytes); call b200_gemm_ws_f32", a_bytes + b_bytes);
  if (!aligned16(workspace)) return fail(B200_EINVAL, "gemm(bf16): workspace must be 16-byte aligned");
  const int64_t Kp = (d.K + 7) / 8 * 8;
  __nv_bfloat16 *a16 = static_cast<__nv_bfloat16 *>(workspace);
  __nv_bfloat16 *b16 = reinterpret_cast<__nv_bfloat16 *>(static_cast<char *>(workspace) + a_bytes);
  auto grid_for = [](int64_t work) {
    int64_t g = (work + 255) / 256;
    return (unsigned)(g > (int64_t)kNumSMs * 16 ? (int64_t)kNumSMs * 16 : (g < 1 ? 1 : g));
  };
  convert_bf16_kernel<<<grid_for(d.M * (Kp / 8)), 256, 0, st>>>(A, a16, d.M, d.K, d.lda, Kp);
  if (int rc = check_launch("convert_bf16(A)")) return rc;
  if (d.trans_b) {
    convert_bf16_kernel<<<grid_for(d.N * (Kp / 8)), 256, 0, st>>>(B, b16, d.N, d.K, d.ldb, Kp);
  } else {
    if ((d.K + 31) / 32 > 65535) return fail(B200_EUNSUPPORTED, "gemm(bf16): K too large for the operand transpose");
    dim3 grid((unsigned)((d.N + 31) / 32), (unsigned)((Kp + 31) / 32));
    convert_bf16_transpose_kernel<<<grid, 256, 0, st>>>(B, b16, d.K, d.N, d.ldb, Kp);
  }
  if (int rc = check_launch("convert_bf16(B)")) return rc;

  const int bn = pick_bn(d.N, false);
  const bool pair = bn == 256 && d.M > BM;
  CUtensorMap ma, mb;
  if (int rc = encode_map_bf16(&ma, a16, (uint64_t)d.K, (uint64_t)d.M, (uint64_t)Kp * 2, 64, BM)) return rc;
  if (int rc = encode_map_bf16(&mb, b16, (uint64_t)d.K, (uint64_t)d.N, (uint64_t)Kp * 2, 64, (uint32_t)(pair ? bn / 2 : bn)))
    return rc;
  GemmParams p{};
  auto aligned_to = [&](int elems) {
    const uintptr_t mask = (uintptr_t)elems * 4 - 1;
    return (reinterpret_cast<uintptr_t>(Y) & mask) == 0 && (!residual || (reinterpret_cast<uintptr_t>(residual) & mask) == 0) &&
           d.ldy % elems == 0;
  };
  p.vec = aligned_to(8) ? 8 : aligned_to(4) ? 4 : 1;
  p.M = d.M;
  p.N = d.N;
  p.num_kb = (int)((d.K + 63) / 64);
  p.num_m_tiles = (int)((d.M + BM - 1) / BM);
  p.num_n_tiles = (int)((d.N + bn - 1) / bn);
  p.batch_inner = 1;
  p.num_tiles = (int64_t)p.num_m_tiles * p.num_n_tiles;
  p.ldy = d.ldy;
  p.epilogue = d.epilogue;
  p.scale = d.scale;
  p.bias = bias;
  p.residual = residual;
  p.Y = Y;
  p.status = device_status_ptr();
  if (!p.status) return fail(B200_ECUDA, "gemm(bf16): device status word unavailable");
  if (pair) {
    p.num_m_tiles = (int)((d.M + 2 * BM - 1) / (2 * BM));
    p.num_tiles_batch = 1;
    return launch_pair<256, false, true>(st, ma, mb, p);
  }
  switch (bn) {
    case 64: return launch_cfg<64, false, false, false, true>(st, ma, mb, p);
    case 128: return launch_cfg<128, false, false, false, true>(st, ma, mb, p);
    default: return launch_cfg<256, false, false, false, true>(st, ma, mb, p);
  }
}

int gemm_tc(cudaStream_t st, const b200_gemm_desc &d_in, const float *A, const float *B, const float *bias,
            const float *residual, float *Y, void *workspace, size_t workspace_bytes) {
  b200_gemm_desc d = d_in;
  if (d.math_mode == B200_MATH_BF16) {
    if (bf16_qualifies(d)) return gemm_tc_bf16(st, d, A, B, bias, residual, Y, workspace, workspace_bytes);
    d.math_mode = B200_MATH_TF32;  // batched operands (attention heads addressed in place) keep the TF32 kernels
  }
  const bool split3 = d.math_mode == B200_MATH_FP32X3;
  // a caller that brings the split workspace anyway gets the pair kernel whatever the size
  const bool pair3 = workspace && aligned16(workspace) && pair3_qualifies(d) &&
                     workspace_bytes >= pair3_workspace_bytes(d);
  // pair kernel: 192-column tiles unless their padding costs more than the slower 128-column instructions
  const bool pair3_wide = ((d.N + 191) / 192) * 192 <= ((d.N + 127) / 128) * 128 * 1.3;
  const int bn = pair3 ? (pair3_wide ? 192 : 128) : pick_bn(d.N, split3);
  // CTA pairs (256 x 256 tiles) for TF32 GEMMs with wide N and at least two row tiles per matrix
  const bool pair = !split3 && bn == 256 && d.M > BM;

  CUtensorMap ma, mb, mb_lo;
  GemmParams p{};
  {
    uint64_t dims[4] = {(uint64_t)d.K, (uint64_t)d.M, 1, 1};
    uint64_t str[3] = {(uint64_t)d.lda * 4, 0, 0};
    const uint64_t fb = (uint64_t)d.lda * 4 * (uint64_t)d.M;
    batch_axis(d.batch_inner, d.a_stride_inner, fb, &dims[2], &str[1], &p.a_bi);
    batch_axis(d.batch_outer, d.a_stride_outer, fb, &dims[3], &str[2], &p.a_bo);
    if (int rc = encode_map(&ma, A, dims, str, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  }
  {
    uint64_t dims[4], str[3];
    uint64_t fb;
    if (d.trans_b) {
      dims[0] = (uint64_t)d.K; dims[1] = (uint64_t)d.N;
      fb = (uint64_t)d.ldb * 4 * (uint64_t)d.N;
    } else {
      dims[0] = (uint64_t)d.N; dims[1] = (uint64_t)d.K;
      fb = (uint64_t)d.ldb * 4 * (uint64_t)d.K;
    }
    str[0] = (uint64_t)d.ldb * 4;
    batch_axis(d.batch_inner, d.b_stride_inner, fb, &dims[2], &str[1], &p.b_bi);
    batch_axis(d.batch_outer, d.b_stride_outer, fb, &dims[3], &str[2], &p.b_bo);
    if (pair3) {
      // split B into the workspace, then describe the two dense copies instead of B itself
      const int64_t rows = d.trans_b ? d.N : d.K, cols = d.trans_b ? d.K : d.N;
      float *b_hi = static_cast<float *>(workspace);
      float *b_lo = reinterpret_cast<float *>(static_cast<char *>(workspace) + align256((size_t)rows * cols * 4));
      const int64_t total4 = rows * (cols / 4);
      int64_t grid = (total4 + 255) / 256;
      if (grid > (int64_t)kNumSMs * 8) grid = (int64_t)kNumSMs * 8;
      split_tf32_kernel<<<(unsigned)grid, 256, 0, st>>>(B, b_hi, b_lo, rows, cols / 4, d.ldb, cols);
      if (int rc = check_launch("split_tf32")) return rc;
      str[0] = (uint64_t)cols * 4;
      const uint32_t box0 = d.trans_b ? BK : 32, box1 = d.trans_b ? (uint32_t)(bn / 2) : BK;
      const CUtensorMapSwizzle sw = d.trans_b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
      if (int rc = encode_map(&mb, b_hi, dims, str, box0, box1, sw)) return rc;
      if (int rc = encode_map(&mb_lo, b_lo, dims, str, box0, box1, sw)) return rc;
    } else if (int rc = encode_map(&mb, B, dims, str, d.trans_b ? BK : 32,
                                   d.trans_b ? (uint32_t)(pair ? bn / 2 : bn) : BK,
                                   d.trans_b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) {
      return rc;
    }
  }
  // Widest access that every output (and residual) row segment is aligned for.
  auto aligned_to = [&](int elems) {
    const uintptr_t mask = (uintptr_t)elems * 4 - 1;
    return (reinterpret_cast<uintptr_t>(Y) & mask) == 0 && (!residual || (reinterpret_cast<uintptr_t>(residual) & mask) == 0) &&
           d.ldy % elems == 0 && d.y_stride_inner % elems == 0 && d.y_stride_outer % elems == 0;
  };
  p.vec = aligned_to(8) ? 8 : aligned_to(4) ? 4 : 1;
  p.M = d.M;
  p.N = d.N;
  p.num_kb = (int)((d.K + BK - 1) / BK);
  p.num_m_tiles = (int)((d.M + BM - 1) / BM);
  p.num_n_tiles = (int)((d.N + bn - 1) / bn);
  p.batch_inner = (int)d.batch_inner;
  p.num_tiles = (int64_t)p.num_m_tiles * p.num_n_tiles * d.batch_outer * d.batch_inner;
  p.ldy = d.ldy;
  p.y_stride_outer = d.y_stride_outer;
  p.y_stride_inner = d.y_stride_inner;
  p.epilogue = d.epilogue;
  p.scale = d.scale;
  p.bias = bias;
  p.residual = residual;
  p.Y = Y;
  p.status = device_status_ptr();
  if (!p.status) return fail(B200_ECUDA, "gemm(tc): device status word unavailable");

  if (pair3) {
    p.num_m_tiles = (int)((d.M + 2 * BM - 1) / (2 * BM));  // 256-row tile pairs
    p.num_tiles_batch = 1;
    if (bn == 192)
      return d.trans_b ? launch_pair3<192, false>(st, ma, mb, mb_lo, p) : launch_pair3<192, true>(st, ma, mb, mb_lo, p);
    return d.trans_b ? launch_pair3<128, false>(st, ma, mb, mb_lo, p) : launch_pair3<128, true>(st, ma, mb, mb_lo, p);
  }
  if (pair) {
    p.num_m_tiles = (int)((d.M + 2 * BM - 1) / (2 * BM));  // 256-row tile pairs
    p.num_tiles_batch = d.batch_outer * d.batch_inner;
    return d.trans_b ? launch_pair<256, false>(st, ma, mb, p) : launch_pair<256, true>(st, ma, mb, p);
  }
  if (d.trans_b) {
    return split3 ? launch_bn<false, true>(st, bn, ma, mb, p) : launch_bn<false, false>(st, bn, ma, mb, p);
  }
  return split3 ? launch_bn<true, true>(st, bn, ma, mb, p) : launch_bn<true, false>(st, bn, ma, mb, p);
}

// ---------------------------------------------------------------------------------------------
// Convolution on the tensor cores (stride 1, any symmetric zero padding, any filter size)
// ---------------------------------------------------------------------------------------------
bool conv2d_tc_supported(const b200_conv_desc &d, const float *X) {
  if (d.math_mode == B200_MATH_FP32) return false;
  if (d.stride_h != 1 || d.stride_w != 1) return false;
  if (d.C % 4 != 0 || d.C < 16) return false;  // TMA: pixel stride C*4 bytes must be a multiple of 16
  if (!aligned16(X)) return false;
  if (d.N > 0x7fffffffLL || d.H > 0x7fffffffLL || d.W > 0x7fffffffLL || d.M > 0x7fffffffLL) return false;
  if (d.KH * d.KW * ((d.C + 31) / 32) > 0x7fffffffLL) return false;
  return true;
}

// Implicit GEMM on gemm_tc_kernel<..., CONV> from an NHWC copy of the input (`xt`) and the repacked filter
// (`wt`: [M][KH*KW][Cp], channels zero-padded to a multiple of 32); writes NCHW. Any output-channel count.
int conv2d_tc_gemm(cudaStream_t st, const b200_conv_desc &d, const float *xt, const float *wt, const float *bias,
                   float *Y, int64_t OH, int64_t OW) {
  const int Cp = (int)((d.C + 31) / 32 * 32);
  const int taps = (int)(d.KH * d.KW);
  const bool split3 = d.math_mode == B200_MATH_FP32X3;
  const int bn = pick_bn(d.M, split3);
  CUtensorMap ma, mb;
  {
    uint64_t dims[4] = {(uint64_t)d.C, (uint64_t)d.W, (uint64_t)d.H, (uint64_t)d.N};
    uint64_t str[3] = {(uint64_t)d.C * 4, (uint64_t)d.W * d.C * 4, (uint64_t)d.H * d.W * d.C * 4};
    if (int rc = encode_map(&ma, xt, dims, str, BK, 8, CU_TENSOR_MAP_SWIZZLE_128B, 8)) return rc;
  }
  {
    uint64_t dims[4] = {(uint64_t)taps * Cp, (uint64_t)d.M, 1, 1};
    uint64_t str[3] = {(uint64_t)taps * Cp * 4, (uint64_t)taps * Cp * 4 * d.M, (uint64_t)taps * Cp * 4 * d.M};
    if (int rc = encode_map(&mb, wt, dims, str, BK, (uint32_t)bn, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  }
  GemmParams p{};
  p.cv.KW = (int)d.KW;
  p.cv.pad_h = (int)d.pad_h;
  p.cv.pad_w = (int)d.pad_w;
  p.cv.OH = (int)OH;
  p.cv.OW = (int)OW;
  p.cv.blocks_w = (int)((OW + 7) / 8);
  p.cv.blocks_per_img = p.cv.blocks_w * (int)((OH + 7) / 8);
  p.cv.cblocks = Cp / 32;
  p.cv.total_blocks = d.N * p.cv.blocks_per_img;
  const int64_t m_tiles = (p.cv.total_blocks + 1) / 2;
  if (m_tiles > 0x7fffffffLL) return fail(B200_EUNSUPPORTED, "conv: too many output tiles");
  p.M = m_tiles * BM;
  p.N = d.M;
  p.num_kb = taps * p.cv.cblocks;
  p.num_m_tiles = (int)m_tiles;
  p.num_n_tiles = (int)((d.M + bn - 1) / bn);
  p.batch_inner = 1;
  p.num_tiles = (int64_t)p.num_m_tiles * p.num_n_tiles;
  p.b_bi = p.b_bo = p.a_bi = p.a_bo = 0;
  p.vec = 1;
  p.epilogue = d.epilogue;
  p.scale = 1.f;
  p.bias = bias;
  p.residual = nullptr;
  p.Y = Y;
  p.status = device_status_ptr();
  if (!p.status) return fail(B200_ECUDA, "conv(tc): device status word unavailable");
  return split3 ? launch_conv_bn<true>(st, bn, ma, mb, p) : launch_conv_bn<false>(st, bn, ma, mb, p);
}

}  // namespace b200

