// Tensor-core Gemm for sm_100a: out[M,N] = act(A[M,K] . W[N,K]^T + bias[N]) + residual[M,N]
// with 16-bit operands (fp16 or bf16), fp32 accumulation in tensor memory and a fused
// epilogue.  Replaces the cuBLASLt calls of lib/Kernels/GPU/Ops.cu:59-120 (mgpuMatmul) and
// :136-234 (mgpuMatmulEx: bias / ReLU / residual epilogues).
//
// Structure (one persistent CTA per SM, 10 warps):
//   warp 0   TMA producer: cp.async.bulk.tensor tiles of A (128 x 64) and W (256 x 64) into
//            a 4-stage ring of 128-byte-swizzled shared memory, completion on mbarriers.
//   warp 1   MMA issuer: one thread issues tcgen05.mma (M=128, N=256, K=16) reading the
//            shared-memory tiles through matrix descriptors; tcgen05.commit releases the
//            stage to the producer and, after the last k-block, hands the accumulator over.
//   warps 2-9 epilogue: tcgen05.ld the 128 x 256 fp32 accumulator out of TMEM (each warp
//            its 32-lane quarter, two warps per quarter splitting the columns), add bias,
//            apply the activation, add the residual, convert.  Each warp stages 32 rows x
//            128 bytes of output in swizzled shared memory and writes it with one TMA
//            store, so global writes are full lines; the residual tile arrives the same
//            way through a TMA load.  (Shapes whose rows are not 16-byte multiples fall
//            back to direct stores.)
// TMEM holds two accumulators (2 x 256 columns) so the epilogue of tile i overlaps the
// mainloop of tile i+1.  Every CTA fetches its own tiles with plain TMA loads and relies on
// L2 for reuse.  All waits are bounded (see ptx_sm100.cuh).
//
// Two variants of the same kernel (template parameter CG):
//   CG = 1  one CTA per 128 x 256 tile (small problems).
//   CG = 2  CTA pairs (cluster of 2, tcgen05 cta_group::2) on 256 x 256 tiles: each CTA
//           stages its 128 rows of A and HALF of the W rows (32 KiB per k-block instead of
//           48), the leader CTA issues one M = 256 MMA for the pair, each CTA keeps its own
//           128 x 256 accumulator and runs its own epilogue.  Tensor-core operand reads and
//           TMA writes compete for shared-memory bandwidth; halving the W bytes per SM is
//           what lifts the mainloop, and the smaller stage allows a 5-deep ring.
#include <cstdlib>
#include <type_traits>

#include "activation.cuh"
#include "ops_common.h"
#include "ptx_sm100.cuh"

namespace mdc {

namespace gemm {
constexpr int BM = 128, BN = 256, BK = 64;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 64 + EPI_WARPS * 32;
constexpr int TMEM_COLS = 512;
constexpr int EPI_BUF_BYTES = 4096;  // 32 rows x 128 bytes, per warp, one for output and one for residual
template <int CG>
struct Cfg {
  static constexpr int B_ROWS = BN / CG;            // W rows this CTA stages per k-block
  static constexpr int B_BYTES = B_ROWS * BK * 2;   // 32 KiB (CG 1) / 16 KiB (CG 2)
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = CG == 2 ? 4 : 3;
  // per epilogue warp: output staging (two buffers for pairs, so a chunk does not wait for
  // the previous chunk's TMA store to drain) + one residual buffer
  static constexpr int OUT_BUFS = CG == 2 ? 2 : 1;
  static constexpr int EPI_WARP_BYTES = (OUT_BUFS + 1) * EPI_BUF_BYTES;
  static constexpr size_t SMEM_BYTES =
      static_cast<size_t>(STAGES) * STAGE_BYTES + EPI_WARPS * EPI_WARP_BYTES + 1024;  // + alignment slack
};
}  // namespace gemm

struct GemmParams {
  int M, N, K;  // K already padded to a multiple of 8
  const float *bias;
  const void *residual;
  void *out;
  int tma_epi;      // output (and residual) rows are 16-byte multiples: TMA-staged epilogue
  int out_vec_ok;   // rows of out / residual can be accessed with 16-byte vectors
  int bias_vec_ok;  // bias is 16-byte aligned
  int num_m_blocks, num_n_blocks;
  int cta_group;  // 1: one CTA per 128 x bn tile; 2: CTA pairs on 256 x bn tiles
  int bn;         // tile width in output columns: 256, 192 or 128 (accumulators stay 256 TMEM columns apart)
  int cw;         // columns per staged output chunk: 64 (16-bit output, 128-byte rows) or 32
  uint32_t *err;
};

template <typename TOut>
__device__ __forceinline__ void store_out8(TOut *dst, const float *v);
template <>
__device__ __forceinline__ void store_out8<float>(float *dst, const float *v) {
  reinterpret_cast<float4 *>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4 *>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store_out8<__half>(__half *dst, const float *v) {
  uint4 o;
  *reinterpret_cast<__half2 *>(&o.x) = __floats2half2_rn(v[0], v[1]);
  *reinterpret_cast<__half2 *>(&o.y) = __floats2half2_rn(v[2], v[3]);
  *reinterpret_cast<__half2 *>(&o.z) = __floats2half2_rn(v[4], v[5]);
  *reinterpret_cast<__half2 *>(&o.w) = __floats2half2_rn(v[6], v[7]);
  *reinterpret_cast<uint4 *>(dst) = o;
}
template <>
__device__ __forceinline__ void store_out8<__nv_bfloat16>(__nv_bfloat16 *dst, const float *v) {
  uint4 o;
  *reinterpret_cast<__nv_bfloat162 *>(&o.x) = __floats2bfloat162_rn(v[0], v[1]);
  *reinterpret_cast<__nv_bfloat162 *>(&o.y) = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<__nv_bfloat162 *>(&o.z) = __floats2bfloat162_rn(v[4], v[5]);
  *reinterpret_cast<__nv_bfloat162 *>(&o.w) = __floats2bfloat162_rn(v[6], v[7]);
  *reinterpret_cast<uint4 *>(dst) = o;
}
__device__ __forceinline__ void load_res8(const __half *src, float *v) {
  const uint4 r = *reinterpret_cast<const uint4 *>(src);
  const __half2 *h = reinterpret_cast<const __half2 *>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void load_res8(const __nv_bfloat16 *src, float *v) {
  const uint4 r = *reinterpret_cast<const uint4 *>(src);
  const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}

// Activation for the Gemm epilogue.  The epilogue runs beside the tensor pipe and must keep
// up with it; its scarce resource is the special-function unit (16 results per clock and SM,
// shared with the 16-bit conversions).  The exact-erf GELU therefore uses ONE special-function
// operation per element:
//   gelu(v) = max(v, 0) - 0.5 |v| erfc(|v| / sqrt 2),     erfc(t) = 2^P(t),
// P a degree-8 polynomial fitted (minimax, t in [0, 5.7]) to log2(erfc(t)); beyond 5.7 the
// erfc term is below 1e-15 |v| and t is clamped.  Against the double-precision erf form the
// result is within 1e-6 absolute and 1.1e-5 relative over [-12, 12] (fp32 evaluation), 50 times
// below the rounding of a 16-bit output.  (The rational form of Abramowitz & Stegun 7.1.26 used
// before needs a reciprocal as well as an exponential.)
__device__ __forceinline__ float ex2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
using ptx::F2;
using ptx::f2;
using ptx::f2_add;
using ptx::f2_fma;
using ptx::f2_get;
using ptx::f2_mul;

__device__ __forceinline__ void gelu_erf_pair(float &va, float &vb) {
  const float aa = fabsf(va), ab = fabsf(vb);
  const F2 T = f2(fminf(aa * 0.70710678f, 5.7f), fminf(ab * 0.70710678f, 5.7f));
#define MDC_C2(x) f2(x, x)
  F2 P = f2_fma(MDC_C2(1.1948015981033677e-06f), T, MDC_C2(-4.147788058617152e-05f));
  P = f2_fma(P, T, MDC_C2(0.0006375535158440471f));
  P = f2_fma(P, T, MDC_C2(-0.005785022862255573f));
  P = f2_fma(P, T, MDC_C2(0.03505704924464226f));
  P = f2_fma(P, T, MDC_C2(-0.1536988914012909f));
  P = f2_fma(P, T, MDC_C2(-0.9163860082626343f));
  P = f2_fma(P, T, MDC_C2(-1.628216028213501f));
  P = f2_fma(P, T, MDC_C2(7.682551768084522e-06f));
#undef MDC_C2
  float pa, pb;
  f2_get(P, pa, pb);
  const F2 E = f2(ex2_approx(pa), ex2_approx(pb));
  const F2 G = f2_fma(f2(-0.5f * aa, -0.5f * ab), E, f2(fmaxf(va, 0.f), fmaxf(vb, 0.f)));
  f2_get(G, va, vb);
}

// Applies the activation to n (even) values in place.
template <int ACT, int N>
__device__ __forceinline__ void act_fast_n(float *v) {
  if constexpr (ACT == kActGeluErf) {
#pragma unroll
    for (int j = 0; j < N; j += 2) gelu_erf_pair(v[j], v[j + 1]);
  } else if constexpr (ACT != kActNone) {
#pragma unroll
    for (int j = 0; j < N; ++j) v[j] = act_apply_t<ACT>(v[j]);
  }
}

template <typename T16, typename TOut, int ACT, int CG>
__global__ void __launch_bounds__(gemm::THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_out,
                    const __grid_constant__ CUtensorMap tmap_res, const GemmParams p) {
  using namespace gemm;
  using namespace ptx;
  using C = Cfg<CG>;
  constexpr int STAGES = C::STAGES, STAGE_BYTES = C::STAGE_BYTES;
  extern __shared__ uint8_t smem_dyn[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full_bar[2], acc_empty_bar[2];
  __shared__ uint64_t res_bar[EPI_WARPS];
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t abort_flag_s;
  volatile uint32_t *abort_flag = &abort_flag_s;

  // 128-byte-swizzled tiles need 1024-byte aligned bases
  uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // CG == 2: the two CTAs of a cluster work on one 256-row tile; rank 0 leads
  const int cta_rank = CG == 2 ? static_cast<int>(cluster_ctarank()) : 0;
  const bool leader = cta_rank == 0;
  const int worker = static_cast<int>(blockIdx.x) / CG, num_workers = static_cast<int>(gridDim.x) / CG;
  // tiles are (CG * 128) rows x bn columns, numbered with the column block running fastest:
  // the workers that run side by side then share their rows of A (read from HBM once, found
  // in L2 by the other column blocks) while W, which is small, stays in L2 throughout
  const int num_m_units = (p.num_m_blocks + CG - 1) / CG;
  const int num_tiles = num_m_units * p.num_n_blocks;
  const int num_kb = (p.K + BK - 1) / BK;
  const int bn = p.bn;  // tile width; this CTA stages bn / CG rows of W per k-block
  const uint32_t stage_tx_bytes = static_cast<uint32_t>(A_BYTES + (bn / CG) * BK * 2);

  if (threadIdx.x == 0) {
    abort_flag_s = 0;
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);   // the leader's arrive.expect_tx (covers both CTAs' bytes)
      mbar_init(&empty_bar[s], 1);  // one tcgen05.commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full_bar[a], 1);
      mbar_init(&acc_empty_bar[a], CG * EPI_WARPS * 32);  // epilogue threads of the whole pair
    }
    for (int w = 0; w < EPI_WARPS; ++w) mbar_init(&res_bar[w], 1);
    mbar_init_fence();
  }
  if (warp == 1) {
    if constexpr (CG == 2) {
      tmem_alloc_cg2(&tmem_slot, TMEM_COLS);
      tmem_relinquish_cg2();
    } else {
      tmem_alloc(&tmem_slot, TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();  // the peer's barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  // Only now, with this CTA's tensor memory allocated, may the next kernel of the chain be set
  // up: a dependent CTA that shared the SM and took tensor-memory columns first would wait for
  // this grid while this CTA waited for its columns.
  pdl_launch_dependents();
  pdl_wait();  // everything above overlaps the previous kernel's tail; operands are read below

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = worker; ok && tile < num_tiles; tile += num_workers) {
        const int m_blk = (tile / p.num_n_blocks) * CG + cta_rank, n_blk = tile % p.num_n_blocks;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            atomicCAS(p.err, 0u, 0x10000000u | static_cast<uint32_t>(stage));
            ok = false;
            break;
          }
          uint8_t *sa = tiles + stage * STAGE_BYTES;
          uint8_t *sb = sa + A_BYTES;
          if constexpr (CG == 2) {
            // both CTAs' copies complete on the LEADER's barrier, which expects the bytes of both
            const uint32_t bar = mapa_u32(smem_u32(&full_bar[stage]), 0);
            if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * stage_tx_bytes);
            tma_load_2d_cg2(sa, &tmap_a, bar, kb * BK, m_blk * BM);
            tma_load_2d_cg2(sb, &tmap_b, bar, kb * BK, n_blk * bn + cta_rank * (bn / 2));
          } else {
            mbar_arrive_expect_tx(&full_bar[stage], stage_tx_bytes);
            tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * BK, m_blk * BM);
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * BK, n_blk * bn);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (lane == 0 && leader) {
      const uint32_t idesc = make_idesc_f16(BM * CG, static_cast<uint32_t>(bn),
                                            std::is_same<T16, __nv_bfloat16>::value, false, false);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = worker; ok && tile < num_tiles; tile += num_workers) {
        if (!mbar_wait(&acc_empty_bar[acc], acc_phase ^ 1, abort_flag)) {
          atomicCAS(p.err, 0u, 0x30000000u | static_cast<uint32_t>(acc));
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            atomicCAS(p.err, 0u, 0x20000000u | static_cast<uint32_t>(stage));
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * STAGE_BYTES);
          const uint64_t a_desc = make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t b_desc = make_smem_desc_sw128(sa + A_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // 16 k-elements = 32 bytes further along the 128-byte swizzled row
            if constexpr (CG == 2)
              umma_f16_ss_cg2(d_tmem, a_desc + static_cast<uint64_t>(2 * k),
                              b_desc + static_cast<uint64_t>(2 * k), idesc, (kb | k) != 0 ? 1u : 0u);
            else
              umma_f16_ss(d_tmem, a_desc + static_cast<uint64_t>(2 * k),
                          b_desc + static_cast<uint64_t>(2 * k), idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // the stage is reusable (in both CTAs) once these MMAs have read it
          if constexpr (CG == 2) {
            umma_commit_cg2(smem_u32(&empty_bar[stage]));
            umma_commit_cg2(mapa_u32(smem_u32(&empty_bar[stage]), 1));
          } else {
            umma_commit(&empty_bar[stage]);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        // accumulator complete: wake the epilogue warps of both CTAs
        if constexpr (CG == 2) {
          umma_commit_cg2(smem_u32(&acc_full_bar[acc]));
          umma_commit_cg2(mapa_u32(smem_u32(&acc_full_bar[acc]), 1));
        } else {
          umma_commit(&acc_full_bar[acc]);
        }
        if ((acc ^= 1) == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int ew = warp - 2;
    const int quarter = warp & 3;   // TMEM lane quarter this warp may access
    const int half_sel = ew >> 2;   // which 128 accumulator columns this warp handles
    TOut *out = static_cast<TOut *>(p.out);
    const T16 *res = static_cast<const T16 *>(p.residual);
    uint8_t *my_out_base = tiles + STAGES * STAGE_BYTES + ew * C::EPI_WARP_BYTES;
    uint8_t *my_res = my_out_base + C::OUT_BUFS * EPI_BUF_BYTES;
    int out_buf = 0;
    uint32_t res_phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    // the accumulator is handed back to the leader's MMA thread, in whichever CTA it lives
    const uint32_t acc_empty_addr0 = mapa_u32(smem_u32(&acc_empty_bar[0]), 0);
    const uint32_t acc_empty_addr1 = mapa_u32(smem_u32(&acc_empty_bar[1]), 0);
    for (int tile = worker; tile < num_tiles; tile += num_workers) {
      const int m_blk = (tile / p.num_n_blocks) * CG + cta_rank, n_blk = tile % p.num_n_blocks;
      // one lane polls, the shuffle releases the others (256 threads would otherwise spin on the
      // barrier word beside the tensor pipe for most of a mainloop)
      if (!mbar_wait_warp(&acc_full_bar[acc], acc_phase, abort_flag)) {
        atomicCAS(p.err, 0u, 0x40000000u | static_cast<uint32_t>(acc));
        break;
      }
      tc_fence_after();
      if (p.tma_epi) {
        // ---- staged path.  The warp owns 32 rows x 128 accumulator columns, read from TMEM in
        // four 32-column pieces; the load of the next piece is in flight while this one goes
        // through bias / activation / residual.  Output leaves in chunks of CW columns
        // (128 bytes per row): swizzled staging buffer -> one TMA store. ----
        // chunk = cw columns; its staged rows are cw * sizeof(TOut) bytes (128, or 64 when a
        // 16-bit tile half is not a multiple of 64 columns), residual rows cw * 2 bytes
        const int cw = p.cw;
        const int SUBS = cw / 32;                          // 32-column pieces per chunk
        const int OUT_ROW_BYTES = cw * static_cast<int>(sizeof(TOut));
        const int RES_ROW_BYTES = cw * 2;                  // residual is 16-bit
        const int half_cols = bn / 2;
        const int row0 = m_blk * BM + quarter * 32;
        const int gcol_base = n_blk * bn + half_sel * half_cols;
        const uint32_t t_base = tmem_base + static_cast<uint32_t>(acc * BN + half_sel * half_cols) +
                                (static_cast<uint32_t>(quarter * 32) << 16);
        // pieces that hold real columns (uniform across the warp; N is a multiple of 4 here)
        const int n_sub = gcol_base >= p.N ? 0 : min(half_cols / 32, (p.N - gcol_base + 31) / 32);
        // 16-byte pieces of a staged row are XOR-swizzled the way TMA expects them:
        // 128-byte rows: piece ^ (row % 8); 64-byte rows: piece ^ ((row / 2) % 4)
        const int swz_out = OUT_ROW_BYTES == 128 ? (lane & 7) : ((lane >> 1) & 3);
        const int swz_res = RES_ROW_BYTES == 128 ? (lane & 7) : ((lane >> 1) & 3);
        uint32_t raw[32];
        if (n_sub > 0) tmem_ld_32x32(t_base, raw);
        bool chunk_ok = true;
        uint8_t *my_out = my_out_base;
#pragma unroll 1
        for (int sub = 0; sub < n_sub; ++sub) {
          const int gcol = gcol_base + sub * 32;
          const int sub_in_chunk = sub % SUBS;
          const int gcol_chunk = gcol - sub_in_chunk * 32;
          if (sub_in_chunk == 0) {
            if (res && lane == 0) {
              mbar_arrive_expect_tx(&res_bar[ew], 32 * RES_ROW_BYTES);
              tma_load_2d(my_res, &tmap_res, &res_bar[ew], gcol_chunk, row0);
            }
            // the TMA store that last used this staging buffer must have finished reading it
            my_out = my_out_base + out_buf * EPI_BUF_BYTES;
            if (lane == 0) tma_store_wait_read<C::OUT_BUFS - 1>();
            __syncwarp();
            if constexpr (C::OUT_BUFS == 2) out_buf ^= 1;
          }
          tmem_ld_wait_regs(raw);
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
          if (sub + 1 < n_sub) tmem_ld_32x32(t_base + (sub + 1) * 32, raw);  // overlaps the math below
          if (p.bias) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (gcol + j < p.N) {
                const float4 b = __ldg(reinterpret_cast<const float4 *>(p.bias + gcol + j));
                v[j] += b.x; v[j + 1] += b.y; v[j + 2] += b.z; v[j + 3] += b.w;
              }
            }
          }
          act_fast_n<ACT, 32>(v);
          if (res) {
            if (sub_in_chunk == 0) {
              if (!mbar_wait_warp(&res_bar[ew], res_phase, abort_flag)) {
                atomicCAS(p.err, 0u, 0x50000000u | static_cast<uint32_t>(ew));
                chunk_ok = false;
                break;
              }
              res_phase ^= 1;
            }
            // this piece is 64 bytes (four 16-byte pieces) of the residual row
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int phys = (sub_in_chunk * 4 + j) ^ swz_res;
              float rv[8];
              load_res8(reinterpret_cast<const T16 *>(my_res + lane * RES_ROW_BYTES + (phys << 4)), rv);
#pragma unroll
              for (int e = 0; e < 8; ++e) v[8 * j + e] += rv[e];
            }
          }
          if constexpr (sizeof(TOut) == 2) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // 32 columns = four 16-byte pieces of the staged row
              const int phys = (sub_in_chunk * 4 + j) ^ swz_out;
              store_out8<TOut>(reinterpret_cast<TOut *>(my_out + lane * OUT_ROW_BYTES + (phys << 4)), v + 8 * j);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<float4 *>(my_out + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                  make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          }
          if (sub_in_chunk == SUBS - 1 || sub + 1 == n_sub) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmap_out, my_out, gcol_chunk, row0);  // rows / columns past M / N are clipped
              tma_store_commit();
            }
          }
        }
        if (!chunk_ok) break;
      } else {
      const int row = m_blk * BM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
#pragma unroll 1
      for (int chunk = 0; chunk < bn / 2 / 32; ++chunk) {
        const int col0 = half_sel * (bn / 2) + chunk * 32;
        const int gcol0 = n_blk * bn + col0;
        if (gcol0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + static_cast<uint32_t>(acc * BN + col0) +
                          (static_cast<uint32_t>(quarter * 32) << 16),
                      r);
        tmem_ld_wait();
        const int ncols = min(32, p.N - gcol0);
        if (ncols == 32 && p.out_vec_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[8 * g + j]);
            if (p.bias) {
              if (p.bias_vec_ok) {
                const float4 b0 = __ldg(reinterpret_cast<const float4 *>(p.bias + gcol0 + 8 * g));
                const float4 b1 = __ldg(reinterpret_cast<const float4 *>(p.bias + gcol0 + 8 * g) + 1);
                v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
                v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += __ldg(p.bias + gcol0 + 8 * g + j);
              }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = act_apply_t<ACT>(v[j]);
            if (row_ok) {
              const size_t off = static_cast<size_t>(row) * p.N + gcol0 + 8 * g;
              if (res) {
                float rv[8];
                load_res8(res + off, rv);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += rv[j];
              }
              store_out8<TOut>(out + off, v);
            }
          }
        } else if (row_ok) {
          // ragged edge or unaligned rows: one element at a time (static register indices)
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (j < ncols) {
              float v = __uint_as_float(r[j]);
              if (p.bias) v += __ldg(p.bias + gcol0 + j);
              v = act_apply_t<ACT>(v);
              const size_t off = static_cast<size_t>(row) * p.N + gcol0 + j;
              if (res) v += static_cast<float>(res[off]);
              out[off] = static_cast<TOut>(v);
            }
          }
        }
      }
      }
      tc_fence_before();
      if constexpr (CG == 2) mbar_arrive_cluster(acc ? acc_empty_addr1 : acc_empty_addr0);
      else mbar_arrive(&acc_empty_bar[acc]);
      if ((acc ^= 1) == 0) acc_phase ^= 1;
    }
    if (lane == 0) tma_store_wait<0>();  // all staged output has left shared memory
  }
  // ------------------------------ teardown ------------------------------
  if (*abort_flag) {
    // a wait gave up: give copies still in flight time to land before the CTA retires
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
  }
  tc_fence_before();
  __syncthreads();
  // neither CTA of a pair may retire (or free tensor memory) while the other can still
  // signal its barriers or read its shared memory
  if constexpr (CG == 2) cluster_sync_all();
  tc_fence_after();
  if (warp == 1) {
    if constexpr (CG == 2) tmem_dealloc_cg2(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------
// The status word the tensor-core kernels write a give-up code into lives in the library
// image (static device storage, zero when the module is loaded), one copy per GPU: no device
// memory is allocated for it, so callers that must not allocate can use and read it too.  Host
// code needs the word's device address, looked up once per device ordinal (a process may
// drive several devices, one at a time).
constexpr int kMaxDevices = 64;
static __device__ uint32_t g_status_word;
static uint32_t *g_err_slots[kMaxDevices] = {nullptr};
static int current_device_index() {
  const int d = device_info().device;
  return (d >= 0 && d < kMaxDevices) ? d : 0;
}

uint32_t *device_error_slot() {
  uint32_t *&slot = g_err_slots[current_device_index()];
  if (!slot) {
    void *sym = nullptr;
    if (!check_cuda(cudaGetSymbolAddress(&sym, g_status_word), "cudaGetSymbolAddress(status word)")) return nullptr;
    slot = static_cast<uint32_t *>(sym);
  }
  return slot;
}

// elem: MGPU_DTYPE_*; swizzle_bytes: 128 or 64 (must equal box_inner * element size)
bool encode_tmap_2d_ex(CUtensorMap *map, const void *base, int32_t elem, uint64_t inner, uint64_t outer,
                       uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle_bytes) {
  const uint64_t gdim[2] = {inner, outer};
  const uint64_t gstr[1] = {row_stride_bytes};
  const uint32_t box[2] = {box_inner, box_outer};
  const uint32_t estr[2] = {1, 1};
  const int before = mgpuGetLastError();
  const int dt = elem == MGPU_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                 : elem == MGPU_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                          : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  mgpuTensorMapEncodeTiled(map, dt, 2, const_cast<void *>(base), gdim, gstr, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE,
                           swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return before != 0 || mgpuGetLastError() == 0;
}

bool encode_tmap_2d(CUtensorMap *map, const void *base, int32_t dtype, uint64_t inner, uint64_t outer,
                    uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  return encode_tmap_2d_ex(map, base, dtype, inner, outer, row_stride_bytes, box_inner, box_outer, 128);
}

template <typename T16, typename TOut, int ACT, int CG>
static void launch_gemm_cg(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &to,
                           const CUtensorMap &tr, const GemmParams &p, int grid, cudaStream_t s) {
  auto kern = gemm_tcgen05_kernel<T16, TOut, ACT, CG>;
  constexpr size_t smem = gemm::Cfg<CG>::SMEM_BYTES;
  static bool attr_set_on[kMaxDevices] = {false};  // the attribute is per device
  bool &attr_set = attr_set_on[current_device_index()];
  if (!attr_set) {
    if (!check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)),
                    "cudaFuncSetAttribute(gemm)"))
      return;
    attr_set = true;
  }
  {
    ProfileScope prof(kCatGemm, s);
    check_cuda(launch_chain(kern, dim3(static_cast<unsigned>(grid)), dim3(gemm::THREADS), smem, s, CG, ta, tb, to, tr, p),
               "launch gemm");
  }
  launched("gemm_tcgen05_kernel");
}

// p.cta_group selects the variant; grid is CTAs (even for pairs)
template <typename T16, typename TOut, int ACT>
static void launch_gemm(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &to,
                        const CUtensorMap &tr, const GemmParams &p, int grid, cudaStream_t s) {
  if (p.cta_group == 2) launch_gemm_cg<T16, TOut, ACT, 2>(ta, tb, to, tr, p, grid, s);
  else launch_gemm_cg<T16, TOut, ACT, 1>(ta, tb, to, tr, p, grid, s);
}

template <typename T16, typename TOut>
static void launch_gemm_act(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &to,
                            const CUtensorMap &tr, const GemmParams &p, int grid, int act, cudaStream_t s) {
  switch (act) {
  case MGPU_ACT_NONE: launch_gemm<T16, TOut, kActNone>(ta, tb, to, tr, p, grid, s); break;
  case MGPU_ACT_RELU: launch_gemm<T16, TOut, kActRelu>(ta, tb, to, tr, p, grid, s); break;
  case MGPU_ACT_GELU_ERF: launch_gemm<T16, TOut, kActGeluErf>(ta, tb, to, tr, p, grid, s); break;
  case MGPU_ACT_GELU_TANH: launch_gemm<T16, TOut, kActGeluTanh>(ta, tb, to, tr, p, grid, s); break;
  default: fail("mgpuMatmulEx16: unknown activation");
  }
}

// CTA pairs whenever there are at least two 128-row blocks; MDC_GEMM_CTA_GROUP=1|2 overrides
// (for measurements).
static int choose_cta_group(int64_t M) {
  static const int forced = [] {
    const char *e = getenv("MDC_GEMM_CTA_GROUP");
    return e ? atoi(e) : 0;
  }();
  if (forced == 1 || forced == 2) return forced;
  return M > gemm::BM ? 2 : 1;
}

// Tile width.  A Gemm takes ceil(tiles / workers) waves of tiles; the last wave is as long as
// the others however few tiles it holds, so for some shapes a narrower tile (more, cheaper
// tiles) wastes less: e.g. M = 32768, N = 768 on 74 CTA pairs is 6 waves of 256-wide tiles
// (5.2 needed) but 7 waves of 192-wide ones (6.9 needed) at 3/4 of the cost each.
// MDC_GEMM_BN=256|192|128 overrides (for measurements).
static int choose_bn(int64_t M, int64_t N, int cta_group, int sms) {
  static const int forced = [] {
    const char *e = getenv("MDC_GEMM_BN");
    return e ? atoi(e) : 0;
  }();
  if (forced == 256 || forced == 192 || forced == 128) return forced;
  const int64_t workers = sms / cta_group > 0 ? sms / cta_group : 1;
  const int64_t m_units = (M + gemm::BM * cta_group - 1) / (gemm::BM * cta_group);
  int best = 256;
  double best_cost = 1e300;
  for (int bn : {256, 192, 128}) {
    const int64_t tiles = m_units * ((N + bn - 1) / bn);
    const int64_t waves = (tiles + workers - 1) / workers;
    // per-tile cost: measured, a 192-wide tile takes about 0.95 of the time of a 256-wide one
    // (the k-block time is set by operand delivery into shared memory, which shrinks only
    // from 32 to 28 KiB per CTA), a 128-wide one about 0.8
    const double cost = static_cast<double>(waves) * (bn == 256 ? 1.0 : bn == 192 ? 0.95 : 0.8);
    if (cost < best_cost * 0.97) {  // prefer the wider tile unless the gain is clear
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

// persistent grid: one worker (CTA or CTA pair) per tile up to the number the device holds
static int gemm_grid(const GemmParams &p, int sms) {
  const int cg = p.cta_group;
  const int64_t tiles = static_cast<int64_t>((p.num_m_blocks + cg - 1) / cg) * p.num_n_blocks;
  if (tiles > 0x7fffffff) return -1;
  const int64_t max_workers = sms / cg;
  if (tiles <= max_workers) return static_cast<int>(tiles * cg);
  // The kernel takes ceil(tiles / workers) rounds whatever the last round holds.  Use the
  // fewest workers that still finish in that many rounds: the SMs left idle draw no power,
  // which the power-capped tensor cores of the others turn into clock (MDC_GEMM_EVEN_WAVES=0
  // uses every SM).
  static const bool even = !(getenv("MDC_GEMM_EVEN_WAVES") && atoi(getenv("MDC_GEMM_EVEN_WAVES")) == 0);
  const int64_t rounds = (tiles + max_workers - 1) / max_workers;
  const int64_t workers = even ? (tiles + rounds - 1) / rounds : max_workers;
  return static_cast<int>(workers * cg);
}

// The whole of mgpuMatmulEx16 after the argument checks: tile choice, tensor maps, launch.
// Shared by every entry point that ends in this Gemm; allocates nothing.
static void matmul16_launch(const char *who, const void *a, const void *w_nk, const float *bias, const void *residual,
                            void *out, int64_t M, int64_t N, int64_t Kp, int32_t dtype, int32_t out_dtype,
                            int32_t act, cudaStream_t s) {
  const DeviceInfo &di = device_info();
  char msg[160];
  auto failf = [&](const char *what) {
    snprintf(msg, sizeof(msg), "%s: %s", who, what);
    fail(msg);
  };
  uint32_t *err = device_error_slot();
  if (!err) return;

  const int cta_group = choose_cta_group(M);
  const int bn = choose_bn(M, N, cta_group, di.sms);
  CUtensorMap ta, tb;
  if (!encode_tmap_2d(&ta, a, dtype, static_cast<uint64_t>(Kp), static_cast<uint64_t>(M),
                      static_cast<uint64_t>(Kp) * 2, gemm::BK, gemm::BM) ||
      !encode_tmap_2d(&tb, w_nk, dtype, static_cast<uint64_t>(Kp), static_cast<uint64_t>(N),
                      static_cast<uint64_t>(Kp) * 2, gemm::BK, bn / cta_group))
    return;

  GemmParams p;
  p.cta_group = cta_group;
  p.bn = bn;
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(Kp);
  p.bias = bias;
  p.residual = residual;
  p.out = out;
  const size_t out_elem = dtype_size(out_dtype);
  const int out_vec = static_cast<int>(16 / out_elem);
  p.out_vec_ok = (N % out_vec == 0) && (N % 8 == 0) && !(reinterpret_cast<uintptr_t>(out) & 15u) &&
                 (!residual || !(reinterpret_cast<uintptr_t>(residual) & 15u));
  p.bias_vec_ok = bias && !(reinterpret_cast<uintptr_t>(bias) & 15u);
  // staged (TMA) epilogue: rows of out / residual must be multiples of 16 bytes and the
  // bias readable as float4
  p.tma_epi = p.out_vec_ok && (!bias || p.bias_vec_ok);
  CUtensorMap to = ta, tr = ta;  // placeholders when the direct-store epilogue is used
  // staged chunks of 64 columns (128-byte rows) for 16-bit output when a tile half is a
  // multiple of 64 columns, else 32 columns
  const uint32_t cw = (out_elem == 2 && (bn / 2) % 64 == 0) ? 64 : 32;
  p.cw = static_cast<int>(cw);
  if (p.tma_epi) {
    if (!encode_tmap_2d_ex(&to, out, out_dtype, static_cast<uint64_t>(N), static_cast<uint64_t>(M),
                           static_cast<uint64_t>(N) * out_elem, cw, 32, static_cast<int>(cw * out_elem)))
      return;
    if (residual && !encode_tmap_2d_ex(&tr, residual, dtype, static_cast<uint64_t>(N), static_cast<uint64_t>(M),
                                       static_cast<uint64_t>(N) * 2, cw, 32, static_cast<int>(cw * 2)))
      return;
  }
  p.num_m_blocks = static_cast<int>((M + gemm::BM - 1) / gemm::BM);
  p.num_n_blocks = static_cast<int>((N + bn - 1) / bn);
  p.err = err;
  const int grid = gemm_grid(p, di.sms);
  if (grid <= 0) { failf("too many tiles"); return; }

  if (dtype == MGPU_DTYPE_F16) {
    if (out_dtype == MGPU_DTYPE_F16) launch_gemm_act<__half, __half>(ta, tb, to, tr, p, grid, act, s);
    else if (out_dtype == MGPU_DTYPE_F32) launch_gemm_act<__half, float>(ta, tb, to, tr, p, grid, act, s);
    else failf("output type must be the operand type or F32");
  } else {
    if (out_dtype == MGPU_DTYPE_BF16) launch_gemm_act<__nv_bfloat16, __nv_bfloat16>(ta, tb, to, tr, p, grid, act, s);
    else if (out_dtype == MGPU_DTYPE_F32) launch_gemm_act<__nv_bfloat16, float>(ta, tb, to, tr, p, grid, act, s);
    else failf("output type must be the operand type or F32");
  }
}
}  // namespace mdc

using namespace mdc;

MDC_API void mgpuMatmulEx16(const void *a, const void *w_nk, const float *bias, const void *residual,
                            void *out, int64_t M, int64_t N, int64_t Kp, int32_t dtype,
                            int32_t out_dtype, int32_t act, void *stream) {
  if (M <= 0 || N <= 0) return;
  const DeviceInfo &di = device_info();
  if (!di.ok) return;
  if (!dtype_is16(dtype)) { fail("mgpuMatmulEx16: dtype must be F16 or BF16"); return; }
  if (Kp <= 0 || (Kp & 7)) { fail("mgpuMatmulEx16: K must be a positive multiple of 8"); return; }
  if (M > 0x7fffffff || N > 0x7fffffff || Kp > 0x7fffffff) { fail("mgpuMatmulEx16: shape too large"); return; }
  if ((reinterpret_cast<uintptr_t>(a) & 15u) || (reinterpret_cast<uintptr_t>(w_nk) & 15u)) {
    fail("mgpuMatmulEx16: operands must be 16-byte aligned");
    return;
  }
  matmul16_launch("mgpuMatmulEx16", a, w_nk, bias, residual, out, M, N, Kp, dtype, out_dtype, act, as_stream(stream));
}

MDC_API uint32_t mgpuOpsCheckDeviceStatus(void *stream) {
  uint32_t *err = device_error_slot();  // an address look-up; allocates nothing
  if (!err) return 0xffffffffu;
  uint32_t h = 0;
  if (!check_cuda(cudaMemcpyAsync(&h, err, sizeof(h), cudaMemcpyDeviceToHost, as_stream(stream)), "read device status"))
    return 0xffffffffu;
  if (!check_cuda(cudaStreamSynchronize(as_stream(stream)), "cudaStreamSynchronize")) return 0xffffffffu;
  if (h != 0) {
    char msg[96];
    snprintf(msg, sizeof(msg), "a tensor-core kernel gave up waiting (code 0x%08x)", h);
    fail(msg);
    cudaMemsetAsync(err, 0, sizeof(uint32_t), as_stream(stream));
  }
  return h;
}

// =========================================================================================
// mgpuMatmulNoAlloc: mgpuMatmul for callers that must not allocate device memory.
//
// mgpuMatmul needs two temporaries (the 16-bit copies of the input and of the transposed
// weight) and takes them from the runtime's device pool, which calls cudaMalloc whenever the
// pool has no fitting block.  Some callers cannot afford that call: a serving loop whose
// latency budget has no room for the device-wide synchronisation cudaMalloc implies, or a
// process in which another component has reserved all device memory up front so that any
// further allocation fails.  For them this entry point does the same computation with the
// temporaries placed in a fixed array that is part of the library image.
//
// * The array is kNoAllocScratchBytes (16 MiB) of device memory per GPU that loads the
//   library, held until the process exits whether the entry point is used or not.
// * Limit: roundup256(M * Kp * 2) + roundup256(N * Kp * 2) <= 16 MiB with Kp = K rounded
//   up to 8 (for example M x N x K = 1024 x 768 x 4096, or 2048 x 512 x 3072).  Larger problems are
//   rejected with the sticky status set and nothing launched.
// * The first call on a device looks the array's device address up
//   (cudaGetSymbolAddress); make that first call before starting any stream capture.
// * All calls on a device share the one array, which keeps whatever the last call left in
//   it.  Everything a call reads from it is written by that call first (the padded operand
//   copies), but two calls that overlap on the GPU (different streams without an ordering
//   between them) race on it: order them.
// * While profiling is off (mgpuOpsProfileBegin creates CUDA events), no cudaMalloc /
//   cudaFree / pool call and no other allocating routine runs on this path.  A kernel that
//   gives up a bounded wait reports through the same status word as every other entry point
//   (mgpuOpsCheckDeviceStatus, which allocates nothing either).
// =========================================================================================
namespace mdc {
constexpr size_t kNoAllocScratchBytes = size_t(16) << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
// host-side cache of the array's device address, per device ordinal
static unsigned char *g_noalloc_ptr[kMaxDevices] = {nullptr};

void cast_rows_padded(const float *src, void *dst, int64_t R, int64_t C, int64_t Cp, int32_t dtype,
                      cudaStream_t s);
}  // namespace mdc

MDC_API void mgpuMatmulNoAlloc(float *input, float *weight, float *bias, float *output, int64_t M,
                               int64_t N, int64_t K, void *stream) {
  if (M <= 0 || N <= 0) return;
  if (K <= 0) { fail("mgpuMatmulNoAlloc: K must be positive"); return; }
  const DeviceInfo &di = device_info();
  if (!di.ok) return;
  if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) { fail("mgpuMatmulNoAlloc: shape too large"); return; }
  const int64_t Kp = (K + 7) / 8 * 8;
  auto up256 = [](size_t b) { return (b + 255) / 256 * 256; };
  const size_t a_bytes = up256(static_cast<size_t>(M) * Kp * 2), w_bytes = up256(static_cast<size_t>(N) * Kp * 2);
  if (a_bytes + w_bytes > kNoAllocScratchBytes) {
    char msg[200];
    snprintf(msg, sizeof(msg),
             "mgpuMatmulNoAlloc: %lld x %lld x %lld needs %zu bytes of scratch, the fixed array holds %zu",
             (long long)M, (long long)N, (long long)K, a_bytes + w_bytes, kNoAllocScratchBytes);
    fail(msg);
    return;
  }
  if (di.device < 0 || di.device >= kMaxDevices) { fail("mgpuMatmulNoAlloc: device ordinal out of range"); return; }
  // set-up, once per device, with that device current: the array's name is only a host-side
  // handle; kernels need the address the runtime resolves for this device
  if (!g_noalloc_ptr[di.device]) {
    void *sym = nullptr;
    if (!check_cuda(cudaGetSymbolAddress(&sym, g_noalloc_scratch), "cudaGetSymbolAddress(scratch)")) return;
    g_noalloc_ptr[di.device] = static_cast<unsigned char *>(sym);
  }
  unsigned char *base = g_noalloc_ptr[di.device];
  void *a16 = base;
  void *w16 = base + a_bytes;
  cudaStream_t s = as_stream(stream);
  cast_rows_padded(input, a16, M, K, Kp, MGPU_DTYPE_F16, s);
  mgpuPackWeight(weight, w16, K, N, MGPU_DTYPE_F16, stream);
  matmul16_launch("mgpuMatmulNoAlloc", a16, w16, bias, nullptr, output, M, N, Kp, MGPU_DTYPE_F16, MGPU_DTYPE_F32,
                  MGPU_ACT_NONE, s);
}
