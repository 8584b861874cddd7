// mgpuConv2d (reference: lib/Kernels/GPU/Ops.cu:238-340, CPU twin lib/Kernels/CPU/Ops.cpp:83-157)
// as an implicit Gemm on the tcgen05 tensor cores: fp32 NCHW tensors and an OIHW filter at the
// boundary, fp16 operands, fp32 accumulation in tensor memory.
//
//   out[n, oc, oh, ow] = sum_k  patch[(n, oh, ow), k] * filter[oc, k]
// with k running over (ic, kh, kw) in an order chosen per shape (see the kernel's template flag).
//
// One CTA computes 128 output pixels x BN output channels.  The patch matrix is never
// written to global memory:
//   * warps 0-7 (two threads per pixel) gather the 64 k-values of their pixel per k-block
//     straight from the NCHW input (a warp's 32 pixels are neighbours along ow, so every load
//     is one coalesced line; all 32 loads of a thread are in flight together), convert them
//     and store their half of the pixel's 128-byte row into shared memory in the
//     128-byte-swizzle layout the tensor core reads; a proxy fence + mbarrier arrive hands the
//     stage to the MMA thread;
//   * warp 8 / lane 0 loads the matching 64 x BN block of the fp16 filter with TMA (plain tile
//     load, 128-byte swizzle; the filter stays in L2);
//   * warp 9 / lane 0 issues tcgen05.mma (M = 128, N = BN, K = 16, four per k-block) and commits
//     each stage back to the producers;
//   * warps 0-7 then read the accumulator (thread = pixel, registers = channels) and write
//     NCHW directly: for a fixed channel a warp's 32 pixels are 128 contiguous bytes, so the
//     stores are whole lines without a transpose.  Bias, postAdd and ReLU are applied here.
// The filter is applied as a cross-correlation (ONNX Conv, oneDNN convolution_forward).
// The reference's GPU path asks cuDNN for CUDNN_CONVOLUTION (a flipped filter, Ops.cu:258),
// which disagrees with its own CPU path; this library follows the CPU path and ONNX.
// With both flags set the result is relu(conv + bias + postAdd), cuDNN's fused form
// (Ops.cu:334-337).
#include <cuda_fp16.h>

#include "ops_common.h"
#include "ptx_sm100.cuh"

namespace mdc {
void cast_rows_padded(const float *src, void *dst, int64_t R, int64_t C, int64_t Cp, int32_t dtype,
                      cudaStream_t s);
bool encode_tmap_2d(CUtensorMap *map, const void *base, int32_t dtype, uint64_t inner, uint64_t outer,
                    uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);

namespace conv {
constexpr int BM = 128;          // output pixels per CTA
constexpr int BK = 64;           // k-elements per stage: one 128-byte swizzled row
constexpr int STAGES = 3;
constexpr int A_BYTES = BM * BK * 2;
constexpr int GATHER_WARPS = 8;  // two threads per pixel row
constexpr int THREADS = (GATHER_WARPS + 2) * 32;  // + filter loader, MMA issuer

struct Params {
  const float *x, *bias, *add;
  float *out;
  int IC, H, W, OC, KH, KW, OH, OW, PHL, PWL, PHR, PWR, SH, SW, DH, DW;
  int tile_bytes;       // MODE 2: size of one staged input tile (two are kept)
  int M, P, K, num_kb;  // pixels in total, pixels per image, IC*KH*KW, k-blocks
  int bn;               // channels per CTA: 32, 64, 128 or 256
  int relu;
  uint32_t *err;
};

inline size_t smem_bytes(int bn, int tile_bytes = 0) {
  return size_t(STAGES) * (A_BYTES + bn * BK * 2) + 2 * size_t(tile_bytes) + 1024;
}
constexpr size_t kMaxSmem = 226 * 1024;  // dynamic part; the static part (barriers) stays under the remaining 1 KiB
}  // namespace conv

// Tap-major order (IC a multiple of 32): k = ((ic / 32) * KH*KW + kh*KW + kw) * 32 + ic % 32, so the
// 32 k-values a gather thread handles share one filter tap (one bounds test, 32 loads a
// channel plane apart) and consecutive k-blocks walk the taps of the same 32 channels, whose
// input lines are then re-served by L1 instead of L2.
// Otherwise k = (ic*KH + kh)*KW + kw (the filter's own order) and every element carries its
// own tap arithmetic.
//
// MODE 0: the filter's own k order, gathered element by element from global memory.
// MODE 1: the k order above, each thread's 32 values loaded from global memory.
// MODE 2: the k order above; the gather warps first stage the input rows the CTA's pixels touch
//         (32 channels at a time, zero padding included, [row][column][channel] in 16 bits) in
//         shared memory with coalesced loads, and every tap of those channels is then a
//         64-byte shared-memory copy per thread, without bounds tests.
template <int MODE>
__global__ void __launch_bounds__(conv::THREADS, MODE == 2 ? 2 : 3)
conv_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_w, const conv::Params p) {
  using namespace conv;
  using namespace ptx;
  constexpr bool TAP_MAJOR = MODE != 0;
  extern __shared__ uint8_t smem_dyn[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
  __shared__ uint32_t tmem_slot, abort_flag_s;
  volatile uint32_t *abort_flag = &abort_flag_s;
  uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bn = p.bn;
  const int stage_bytes = A_BYTES + bn * BK * 2;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * bn;

  if (threadIdx.x == 0) {
    abort_flag_s = 0;
    tma_prefetch_desc(&tmap_w);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], GATHER_WARPS + 1);  // one arrive per gather warp + the filter loader's expect_tx
      mbar_init(&empty_bar[s], 1);      // one tcgen05.commit
    }
    mbar_init(&acc_bar, 1);
    mbar_init_fence();
  }
  if (warp == GATHER_WARPS) {
    tmem_alloc(&tmem_slot, static_cast<uint32_t>(bn));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  pdl_launch_dependents();  // after this CTA holds its tensor memory (see the Gemm kernel)
  pdl_wait();

  if (warp < GATHER_WARPS) {
    // ---------------- gather: two threads per output pixel, 32 k-values each ----------------
    const int row = threadIdx.x & (BM - 1);
    const int half = threadIdx.x >> 7;  // which 32 of the stage's 64 k-values
    const int m = m0 + row;
    const bool live = m < p.M;
    int n = 0, ih0 = 0, iw0 = 0, pix = 0;
    if (live) {
      n = m / p.P;
      pix = m - n * p.P;
      const int oh = pix / p.OW, ow = pix - oh * p.OW;
      ih0 = oh * p.SH - p.PHL;
      iw0 = ow * p.SW - p.PWL;
    }
    const float *img = p.x + static_cast<int64_t>(n) * p.IC * p.H * p.W;
    // pixels whose whole window lies inside the image skip the bounds tests
    const bool interior = live && ih0 >= 0 && iw0 >= 0 && ih0 + (p.KH - 1) * p.DH < p.H &&
                          iw0 + (p.KW - 1) * p.DW < p.W;
    const int khw = p.KH * p.KW, hw = p.H * p.W;
    const int pix_off = ih0 * p.W + iw0;
    const uint32_t row_off = static_cast<uint32_t>(row) * 128u;
    const uint32_t swz = static_cast<uint32_t>(row & 7);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    // loads of k-block kb into registers (no shared memory involved yet)
    auto gather = [&](int kb, float (&v)[32]) __attribute__((always_inline)) {
      const int k0 = kb * BK + half * 32;
      if constexpr (TAP_MAJOR) {
        const int q = k0 >> 5;  // this thread's group of 32 k-values = (channel block, tap)
        const int icb = q / khw, tap = q - icb * khw;
        const int ic0 = icb * 32;
        const int kh = tap / p.KW, kw = tap - kh * p.KW;
        const int ih = ih0 + kh * p.DH, iw = iw0 + kw * p.DW;
        if (live && k0 < p.K && static_cast<unsigned>(ih) < static_cast<unsigned>(p.H) &&
            static_cast<unsigned>(iw) < static_cast<unsigned>(p.W)) {
          const float *src = img + ic0 * hw + ih * p.W + iw;
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __ldg(src + j * hw);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
      } else if (k0 >= p.K || !live) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0.f;
      } else {
        int ic = k0 / khw;
        int r = k0 - ic * khw;
        int kh = r / p.KW;
        int kw = r - kh * p.KW;
        // in batches of 16: offsets (pure integer work, no branches), then the loads, all in
        // flight together; elements outside the image or beyond K read offset 0 of the image
        // and are zeroed afterwards
        uint32_t valid = 0;
#pragma unroll
        for (int b = 0; b < 32; b += 16) {
          int off[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int dh = kh * p.DH, dw = kw * p.DW;
            const bool inside = static_cast<unsigned>(ih0 + dh) < static_cast<unsigned>(p.H) &
                                static_cast<unsigned>(iw0 + dw) < static_cast<unsigned>(p.W);
            const bool in = (k0 + b + j < p.K) & (interior | inside);
            off[j] = in ? ic * hw + dh * p.W + dw + pix_off : 0;
            valid |= (in ? 1u : 0u) << (b + j);
            const bool wrap_w = ++kw == p.KW;
            kw = wrap_w ? 0 : kw;
            kh += wrap_w ? 1 : 0;
            const bool wrap_h = kh == p.KH;
            kh = wrap_h ? 0 : kh;
            ic += wrap_h ? 1 : 0;
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) v[b + j] = __ldg(img + off[j]);
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (valid >> j) & 1u ? v[j] : 0.f;
      }
    };
    // waits for the stage to be free, then converts and stores the row and hands it over
    auto put = [&](float (&v)[32]) __attribute__((always_inline)) -> bool {
      if (!mbar_wait_warp(&empty_bar[stage], phase ^ 1, abort_flag)) {
        atomicCAS(p.err, 0u, 0x50000000u | static_cast<uint32_t>(stage));
        return false;
      }
      uint8_t *sa = tiles + stage * stage_bytes;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const __half2 h0 = __floats2half2_rn(v[c * 8 + 0], v[c * 8 + 1]), h1 = __floats2half2_rn(v[c * 8 + 2], v[c * 8 + 3]);
        const __half2 h2 = __floats2half2_rn(v[c * 8 + 4], v[c * 8 + 5]), h3 = __floats2half2_rn(v[c * 8 + 6], v[c * 8 + 7]);
        uint4 q;
        q.x = *reinterpret_cast<const uint32_t *>(&h0);
        q.y = *reinterpret_cast<const uint32_t *>(&h1);
        q.z = *reinterpret_cast<const uint32_t *>(&h2);
        q.w = *reinterpret_cast<const uint32_t *>(&h3);
        // 128-byte swizzle: 16-byte chunk c of row r lives at chunk (c ^ (r & 7))
        const uint32_t chunk = static_cast<uint32_t>(half * 4 + c);
        *reinterpret_cast<uint4 *>(sa + row_off + ((chunk ^ swz) << 4)) = q;
      }
      fence_proxy_async_smem();  // the tensor core reads these rows through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_bar[stage]);
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
      return true;
    };
    if constexpr (MODE == 2) {
      // Rows of the padded input are numbered g = image * Hp + padded row; the CTA's pixels touch
      // the rows [g_base, g_base + span) (the padding rows between two images included).
      const int Hp = p.H + p.PHL + p.PHR, Wp = p.W + p.PWL + p.PWR;
      const int ml = min(m0 + BM - 1, p.M - 1);
      const int nf = m0 / p.P, ohf = (m0 - nf * p.P) / p.OW;
      const int nl = ml / p.P, ohl = (ml - nl * p.P) / p.OW;
      const int g_base = nf * Hp + ohf * p.SH;
      const int span = nl * Hp + ohl * p.SH + (p.KH - 1) * p.DH - g_base + 1;
      uint8_t *T = tiles + STAGES * stage_bytes;
      // the host sized the tiles from an upper bound of span; never write past them
      if (span * Wp * 64 > p.tile_bytes) {
        atomicCAS(p.err, 0u, 0x54000000u);
        ok = false;
      }
      // this thread's pixel, clamped to the last real one so that every read stays in the tile
      const int mc = min(m, p.M - 1);
      const int nc = mc / p.P, pc = mc - nc * p.P, ohc = pc / p.OW, owc = pc - ohc * p.OW;
      const int g_pix = nc * Hp + ohc * p.SH - g_base, iw_pix = owc * p.SW;
      const int ngroups = p.K >> 5;
      int staged_upto = -1;
      // one thread per position (row, column) and all 32 channels: neighbouring lanes hold
      // neighbouring columns, so each of the 32 loads is a coalesced line and all of them are in
      // flight together; the values leave as four 16-byte stores
      auto stage_tile = [&](int icb) {
        uint8_t *Tb = T + (icb & 1) * p.tile_bytes;
        const int positions = span * Wp;
        for (int pos = threadIdx.x; pos < positions; pos += GATHER_WARPS * 32) {
          const int g = pos / Wp, iwp = pos - g * Wp;
          const int G = g + g_base, nn = G / Hp, ih = G - nn * Hp - p.PHL, iw = iwp - p.PWL;
          float e[32];
          if (static_cast<unsigned>(ih) < static_cast<unsigned>(p.H) && static_cast<unsigned>(iw) < static_cast<unsigned>(p.W)) {
            const float *src = p.x + (static_cast<int64_t>(nn) * p.IC + icb * 32) * hw + ih * p.W + iw;
#pragma unroll
            for (int j = 0; j < 32; ++j) e[j] = __ldg(src + j * hw);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) e[j] = 0.f;
          }
          uint8_t *dst = Tb + pos * 64;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const __half2 h0 = __floats2half2_rn(e[c * 8 + 0], e[c * 8 + 1]), h1 = __floats2half2_rn(e[c * 8 + 2], e[c * 8 + 3]);
            const __half2 h2 = __floats2half2_rn(e[c * 8 + 4], e[c * 8 + 5]), h3 = __floats2half2_rn(e[c * 8 + 6], e[c * 8 + 7]);
            uint4 q;
            q.x = *reinterpret_cast<const uint32_t *>(&h0);
            q.y = *reinterpret_cast<const uint32_t *>(&h1);
            q.z = *reinterpret_cast<const uint32_t *>(&h2);
            q.w = *reinterpret_cast<const uint32_t *>(&h3);
            // the four 16-byte pieces of a position are XOR-ed with its column, which spreads a
            // warp's accesses over the banks
            *reinterpret_cast<uint4 *>(dst + ((c ^ (iwp & 3)) << 4)) = q;
          }
        }
      };
      for (int kb = 0; kb < p.num_kb; ++kb) {
        // every gather warp passes the same barriers whatever happened to its waits, so a
        // warp that gave up cannot strand the others
        const int need = min(2 * kb + 1, ngroups - 1) / khw;
        while (staged_upto < need) {
          asm volatile("bar.sync 1, %0;" ::"n"(GATHER_WARPS * 32) : "memory");  // the buffer's last readers are done
          if (ok) stage_tile(staged_upto + 1);
          ++staged_upto;
          asm volatile("bar.sync 1, %0;" ::"n"(GATHER_WARPS * 32) : "memory");
        }
        if (!ok) continue;
        if (!mbar_wait_warp(&empty_bar[stage], phase ^ 1, abort_flag)) {
          atomicCAS(p.err, 0u, 0x50000000u | static_cast<uint32_t>(stage));
          ok = false;
          continue;
        }
        uint8_t *sa = tiles + stage * stage_bytes;
        const int q = 2 * kb + half;
        uint4 piece[4];
        if (q < ngroups) {
          const int icb = q / khw, tap = q - icb * khw;
          const int kh = tap / p.KW, kw = tap - kh * p.KW;
          const int iwp = iw_pix + kw * p.DW;
          const uint8_t *src = T + (icb & 1) * p.tile_bytes + ((g_pix + kh * p.DH) * Wp + iwp) * 64;
#pragma unroll
          for (int c = 0; c < 4; ++c) piece[c] = *reinterpret_cast<const uint4 *>(src + ((c ^ (iwp & 3)) << 4));
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) piece[c] = make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
          *reinterpret_cast<uint4 *>(sa + row_off + ((static_cast<uint32_t>(half * 4 + c) ^ swz) << 4)) = piece[c];
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_bar[stage]);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    } else {
      for (int kb = 0; kb < p.num_kb; ++kb) {
        float v[32];
        gather(kb, v);
        if (!put(v)) { ok = false; break; }
      }
    }

    // ------- epilogue: thread = pixel, registers = channels; the two threads of a pixel -------
    // ------- take alternate groups of 32 channels                                       -------
    // (ok is uniform within a warp: the waits above are warp-wide)
    if (ok && !mbar_wait_warp(&acc_bar, 0, abort_flag)) {
      atomicCAS(p.err, 0u, 0x52000000u);
      ok = false;
    }
    if (ok) {
      tc_fence_after();
      const int64_t out_base = static_cast<int64_t>(n) * p.OC * p.P + pix;
      // a warp may only read the 32 tensor-memory lanes (warp % 4) * 32 ...
      const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
      // 16 channels at a time: bias and postAdd values are fetched as one batch of independent
      // loads while the accumulator load is in flight, never one load between two stores
      for (int c32 = half * 32; c32 < bn && n0 + c32 < p.OC; c32 += 64) {
#pragma unroll
        for (int c0 = c32; c0 < c32 + 32; c0 += 16) {
          const int oc0 = n0 + c0;
          if (oc0 >= p.OC) break;  // uniform across the warp
          uint32_t acc[16];
          tmem_ld_32x16(tmem_base + lane_base + static_cast<uint32_t>(c0), acc);
          float extra[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) extra[j] = (p.bias && oc0 + j < p.OC) ? __ldg(p.bias + oc0 + j) : 0.f;
          if (p.add && live) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (oc0 + j < p.OC) extra[j] += __ldg(p.add + out_base + static_cast<int64_t>(oc0 + j) * p.P);
          }
          tmem_ld_wait_regs(acc);
          if (live) {
            float *dst = p.out + out_base + static_cast<int64_t>(oc0) * p.P;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (oc0 + j < p.OC) {
                float v = __uint_as_float(acc[j]) + extra[j];
                if (p.relu) v = fmaxf(v, 0.f);
                dst[static_cast<int64_t>(j) * p.P] = v;
              }
            }
          }
        }
      }
    }
  } else if (warp == GATHER_WARPS) {
    // ------------------------- filter loader -------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t tx = static_cast<uint32_t>(bn * BK * 2);
      for (int kb = 0; kb < p.num_kb; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
          atomicCAS(p.err, 0u, 0x51000000u | static_cast<uint32_t>(stage));
          break;
        }
        mbar_arrive_expect_tx(&full_bar[stage], tx);
        tma_load_2d(tiles + stage * stage_bytes + A_BYTES, &tmap_w, &full_bar[stage], kb * BK, n0);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------- MMA issuer -------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(BM, static_cast<uint32_t>(bn), false, false, false);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < p.num_kb; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
          atomicCAS(p.err, 0u, 0x53000000u | static_cast<uint32_t>(stage));
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(tiles + stage * stage_bytes);
        const uint64_t a_desc = make_smem_desc_sw128(sa, 16, 1024);
        const uint64_t b_desc = make_smem_desc_sw128(sa + A_BYTES, 16, 1024);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          umma_f16_ss(tmem_base, a_desc + static_cast<uint64_t>(2 * k), b_desc + static_cast<uint64_t>(2 * k),
                      idesc, (kb | k) != 0 ? 1u : 0u);
        umma_commit(&empty_bar[stage]);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (ok) umma_commit(&acc_bar);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == GATHER_WARPS) tmem_dealloc(tmem_base, static_cast<uint32_t>(bn));
}


// OIHW fp32 filter -> fp16 [OC][((ic / 32) * taps + tap) * 32 + ic % 32] (the k order of the
// TAP_MAJOR kernel); IC is a multiple of 32
__global__ void __launch_bounds__(256) pack_filter_tap_major(const float *__restrict__ w, __half *__restrict__ out,
                                                             int OC, int IC, int taps) {
  const int64_t total = static_cast<int64_t>(OC) * IC * taps;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int lane_ic = static_cast<int>(i & 31);
    const int64_t t = i >> 5;
    const int tap = static_cast<int>(t % taps);
    const int64_t u = t / taps;
    const int icb = static_cast<int>(u % (IC / 32));
    const int64_t oc = u / (IC / 32);
    out[i] = __float2half_rn(__ldg(w + (oc * IC + icb * 32 + lane_ic) * taps + tap));
  }
}

}  // namespace mdc

using namespace mdc;

MDC_API void mgpuConv2d(float *input, float *weight, float *bias, float *output, float *postAdd, int64_t N,
                        int64_t IC, int64_t H, int64_t W, int64_t OC, int64_t KH, int64_t KW, int64_t OH,
                        int64_t OW, int64_t PHL, int64_t PWL, int64_t PHR, int64_t PWR, int64_t SH, int64_t SW,
                        int64_t DH, int64_t DW, bool hasPostAdd, bool hasContainRelu, void *stream) {
  if (N <= 0 || OC <= 0 || OH <= 0 || OW <= 0) return;
  if (IC <= 0 || H <= 0 || W <= 0 || KH <= 0 || KW <= 0 || SH <= 0 || SW <= 0 || DH <= 0 || DW <= 0 ||
      PHL < 0 || PWL < 0 || PHR < 0 || PWR < 0) {
    fail("mgpuConv2d: sizes, strides and dilations must be positive, paddings non-negative");
    return;
  }
  // the caller's output extent must be one its geometry can produce
  if ((OH - 1) * SH + (KH - 1) * DH + 1 > H + PHL + PHR || (OW - 1) * SW + (KW - 1) * DW + 1 > W + PWL + PWR) {
    fail("mgpuConv2d: output extent does not fit the padded input");
    return;
  }
  if (hasPostAdd && !postAdd) { fail("mgpuConv2d: hasPostAdd without a postAdd tensor"); return; }
  const int64_t M = N * OH * OW, K = IC * KH * KW;
  // 32-bit index arithmetic inside the kernel
  if (M > INT32_MAX - conv::BM || K > (1 << 24) || OC > (1 << 20) || IC * H * W > INT32_MAX ||
      (H + PHL + PHR + KH * DH) * W > INT32_MAX) {
    fail("mgpuConv2d: shape exceeds this library's index range");
    return;
  }
  if (!device_info().ok) return;
  cudaStream_t s = as_stream(stream);
  const int64_t Kp = (K + 7) / 8 * 8;  // filter rows padded to 16-byte multiples for TMA
  void *w16 = mgpuMemAllocAsync(static_cast<uint64_t>(OC) * Kp * 2, stream);
  if (!w16) return;
  const bool tap_major = IC % 32 == 0;
  if (tap_major) {
    const int64_t total = OC * K;
    const int64_t blocks = (total + 255) / 256;
    pack_filter_tap_major<<<static_cast<unsigned>(blocks < 4096 ? blocks : 4096), 256, 0, s>>>(
        weight, static_cast<__half *>(w16), int(OC), int(IC), int(KH * KW));
    check_cuda(cudaGetLastError(), "launch pack_filter_tap_major");
    launched("mdc_pack_filter");
  } else {
    cast_rows_padded(weight, w16, OC, K, Kp, MGPU_DTYPE_F16, s);
  }

  conv::Params p;
  p.x = input, p.bias = bias, p.add = hasPostAdd ? postAdd : nullptr, p.out = output;
  p.IC = int(IC), p.H = int(H), p.W = int(W), p.OC = int(OC), p.KH = int(KH), p.KW = int(KW);
  p.OH = int(OH), p.OW = int(OW), p.PHL = int(PHL), p.PWL = int(PWL), p.SH = int(SH), p.SW = int(SW);
  p.DH = int(DH), p.DW = int(DW), p.PHR = int(PHR), p.PWR = int(PWR), p.tile_bytes = 0;
  p.M = int(M), p.P = int(OH * OW), p.K = int(K), p.num_kb = int((K + conv::BK - 1) / conv::BK);
  // channels per CTA: wide tiles gather each pixel's patch fewer times, but the grid should
  // still cover the SMs
  p.bn = OC <= 32 ? 32 : OC <= 64 ? 64 : OC <= 128 ? 128 : 256;
  const int64_t m_tiles = (M + conv::BM - 1) / conv::BM;
  while (p.bn > 64 && m_tiles * ((OC + p.bn - 1) / p.bn) < device_info().sms) p.bn /= 2;
  p.relu = hasContainRelu ? 1 : 0;
  p.err = device_error_slot();
  CUtensorMap tw;
  // rows beyond OC and k beyond Kp read as zero
  if (p.err && encode_tmap_2d(&tw, w16, MGPU_DTYPE_F16, static_cast<uint64_t>(Kp), static_cast<uint64_t>(OC),
                              static_cast<uint64_t>(Kp) * 2, conv::BK, static_cast<uint32_t>(p.bn))) {
    // Staged mode: an upper bound of the padded input rows one CTA's 128 pixels touch.  The
    // pixels cross at most `turns` row boundaries, each a step of SH rows or, between two
    // images, of the rows left over at the bottom of one image and the top of the next.
    int mode = tap_major ? 1 : 0;
    if (tap_major && getenv("MDC_CONV_DIRECT") == nullptr) {
      const int64_t Hp = H + PHL + PHR, Wp = W + PWL + PWR;
      const int64_t turns = (conv::BM - 2 + OW) / OW;
      const int64_t crossings = turns < (turns + OH - 1) / OH ? turns : (turns + OH - 1) / OH;
      const int64_t cross_step = Hp - (OH - 1) * SH > SH ? Hp - (OH - 1) * SH : SH;
      const int64_t span = (turns - crossings) * SH + crossings * cross_step + (KH - 1) * DH + 1;
      const int64_t tile_bytes = span * Wp * 64;
      // only when two CTAs still fit on an SM: alone, a CTA cannot hide its staging loads
      // (measured: 32x64x56x56 -> 64 takes 90 us staged with one CTA per SM, 53 us direct;
      // 32x256x14x14 -> 256 takes 61 us staged with two CTAs per SM, 66 us direct)
      if (2 * (conv::smem_bytes(p.bn, static_cast<int>(tile_bytes < (1 << 20) ? tile_bytes : (1 << 20))) + 1024) <= conv::kMaxSmem) {
        mode = 2;
        p.tile_bytes = static_cast<int>(tile_bytes);
      }
    }
    const size_t smem = conv::smem_bytes(p.bn, p.tile_bytes);
    // dynamic shared memory limit, raised once per device
    static int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
      const int limit = static_cast<int>(conv::kMaxSmem);
      if (check_cuda(cudaFuncSetAttribute(conv_tcgen05_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, limit),
                     "cudaFuncSetAttribute(conv)") &&
          check_cuda(cudaFuncSetAttribute(conv_tcgen05_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, limit),
                     "cudaFuncSetAttribute(conv)") &&
          check_cuda(cudaFuncSetAttribute(conv_tcgen05_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, limit),
                     "cudaFuncSetAttribute(conv)"))
        attr_dev = dev;
    }
    const dim3 grid(static_cast<unsigned>((M + conv::BM - 1) / conv::BM),
                    static_cast<unsigned>((OC + p.bn - 1) / p.bn));
    {
      ProfileScope prof(kCatGemm, s);
      if (mode == 2) conv_tcgen05_kernel<2><<<grid, conv::THREADS, smem, s>>>(tw, p);
      else if (mode == 1) conv_tcgen05_kernel<1><<<grid, conv::THREADS, smem, s>>>(tw, p);
      else conv_tcgen05_kernel<0><<<grid, conv::THREADS, smem, s>>>(tw, p);
      check_cuda(cudaGetLastError(), "launch conv_tcgen05_kernel");
    }
    launched("conv_tcgen05_kernel");
  }
  mgpuMemFreeAsync(w16, stream);
}
