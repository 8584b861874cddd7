// Fused multi-head attention for sm_100a, head_dim 64, fp16 / bf16:
//   out = softmax(Q.K^T / sqrt(d) + mask) . V        per (batch, head)
// on the packed QKV Gemm output [tokens, 3, heads, 64].  Replaces the vendored
// FusedMHARunnerFP16v2 (precompiled sm_70..sm_89 cubins) that the reference layer calls at
// lib/Kernels/GPU/LLM.cu:79-81; masks: key padding from per-sequence lengths and, optionally,
// causal.
//
// One CTA handles 128 queries of one (batch, head) and walks the keys in tiles of 128
// (flash-style online softmax; tiles that are fully masked are skipped):
//   warp 4, one thread   TMA loads of the Q / K / V tiles (128 x 64, 128-byte swizzle) and
//                        the two tcgen05.mma groups per key tile:
//                          S = Q.K^T   (M=128, N=128, K=64)  -> TMEM columns [0,128)
//                          O_t = P.V   (M=128, N=64, K=128)  -> TMEM columns [64,128)
//                        P (16-bit, two keys per 32-bit column) is written by the softmax
//                        threads over S columns [0,64) they have already consumed and is
//                        the A operand of the second MMA straight from tensor memory.
//                        V is used as it lies in memory (keys x head_dim, an MN-major B
//                        operand), so no transpose pass is needed.
//   warps 0-3            one thread per query row: tcgen05.ld the scores, running max and
//                        sum in fp32 (exp2 with log2(e)/sqrt(d) folded in), P stored back
//                        into tensor memory (tcgen05.st), then the partial product O_t is
//                        read back and accumulated in registers with the usual rescaling.
// Shared memory is 49 KiB (Q, K, V tiles only) and TMEM 128 columns per CTA, so three CTAs
// share an SM and overlap each other's load / MMA / softmax phases.  Every wait is bounded.
#include <type_traits>

#include "ops_common.h"
#include "ptx_sm100.cuh"

namespace mdc {

namespace attn {
constexpr int BQ = 128, BKV = 128, D = 64;
constexpr int TILE_BYTES = 128 * D * 2;  // 16 KiB: one 128 x 64 16-bit tile
constexpr int THREADS = 160;
constexpr int TMEM_COLS = 128;
constexpr int S_COL = 0, P_COL = 0, O_COL = 64;
constexpr int CTAS_PER_SM = 3;
constexpr size_t SMEM_BYTES = 3 * TILE_BYTES + 1024;
}  // namespace attn

struct AttnParams {
  const int32_t *seq_lens;  // [batch] or nullptr
  void *out;                // [batch*seq, heads*64]
  int batch, seq, heads;
  int causal;
  float scale_log2e;  // log2(e) / sqrt(d)
  uint32_t *err;
};

template <typename T16>
__device__ __forceinline__ uint32_t pack16(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack16<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack16<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}

// One unit of work: 128 queries of one (sequence, head).  Decoded identically by the control
// thread and the softmax threads, so both walk the same sequence of key tiles.
struct AttnItem {
  int q0, head, b, row_base, kv_end, n_kv;
};
__device__ __forceinline__ AttnItem attn_item(const AttnParams &p, int item, int q_tiles) {
  AttnItem it;
  const int qt = item % q_tiles;
  const int rest = item / q_tiles;
  it.head = rest % p.heads;
  it.b = rest / p.heads;
  it.q0 = qt * attn::BQ;
  it.row_base = it.b * p.seq;
  const int len = p.seq_lens ? min(max(p.seq_lens[it.b], 0), p.seq) : p.seq;
  it.kv_end = p.causal ? min(len, it.q0 + attn::BQ) : len;  // keys this query tile can see: [0, kv_end)
  it.n_kv = (it.kv_end + attn::BKV - 1) / attn::BKV;
  return it;
}

__device__ __forceinline__ float ex2_fast(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// Persistent: each CTA walks work items item = blockIdx.x, + gridDim.x, ...; the key tiles of
// all its items form one sequence of steps t = 0, 1, ..., and every barrier completes once
// per step (parity t & 1), so loads for step t+1 (of the same or of the next item) are issued
// while step t is still in its softmax: K (and the next item's Q) as soon as S = Q.K^T of
// step t has been computed, V as soon as P.V of step t has.
template <typename T16>
__global__ void __launch_bounds__(attn::THREADS, attn::CTAS_PER_SM)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_qkv, const AttnParams p) {
  using namespace attn;
  using namespace ptx;
  extern __shared__ uint8_t smem_dyn[];
  __shared__ uint64_t bar_q, bar_k, bar_v, bar_s_full, bar_p_ready, bar_o_full, bar_o_read;
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t abort_flag_s;
  volatile uint32_t *abort_flag = &abort_flag_s;

  uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
  uint8_t *sQ = tiles, *sK = tiles + TILE_BYTES, *sV = tiles + 2 * TILE_BYTES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tiles = (p.seq + BQ - 1) / BQ;
  const int n_items = q_tiles * p.heads * p.batch;
  const int hd = p.heads * D;

  if (threadIdx.x == 0) {
    abort_flag_s = 0;
    tma_prefetch_desc(&tmap_qkv);
    mbar_init(&bar_q, 1);
    mbar_init(&bar_k, 1);
    mbar_init(&bar_v, 1);
    mbar_init(&bar_s_full, 1);
    mbar_init(&bar_p_ready, 128);
    mbar_init(&bar_o_full, 1);
    mbar_init(&bar_o_read, 128);
    mbar_init_fence();
  }
  if (warp == 4) {
    tmem_alloc(&tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  pdl_launch_dependents();  // after this CTA holds its tensor memory (see the Gemm kernel)
  pdl_wait();  // set-up above overlaps the previous kernel's tail; QKV is read below

  if (warp == 4) {
    // ------------------------------ loads + MMA issue ------------------------------
    if (lane == 0) {
      constexpr bool kBf16 = std::is_same<T16, __nv_bfloat16>::value;
      constexpr uint32_t idesc_s = make_idesc_f16(BQ, BKV, kBf16, false, false);
      constexpr uint32_t idesc_o = make_idesc_f16(BQ, D, kBf16, false, true);  // V is MN-major
      const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      auto load_q = [&](const AttnItem &it) {
        mbar_arrive_expect_tx(&bar_q, TILE_BYTES);
        tma_load_2d(sQ, &tmap_qkv, &bar_q, it.head * D, it.row_base + it.q0);
      };
      auto load_k = [&](const AttnItem &it, int j) {
        mbar_arrive_expect_tx(&bar_k, TILE_BYTES);
        tma_load_2d(sK, &tmap_qkv, &bar_k, hd + it.head * D, it.row_base + j * BKV);
      };
      auto load_v = [&](const AttnItem &it, int j) {
        mbar_arrive_expect_tx(&bar_v, TILE_BYTES);
        tma_load_2d(sV, &tmap_qkv, &bar_v, 2 * hd + it.head * D, it.row_base + j * BKV);
      };
      // first item with at least one visible key
      int item = blockIdx.x;
      AttnItem cur{};
      while (item < n_items && (cur = attn_item(p, item, q_tiles)).n_kv == 0) item += gridDim.x;
      uint32_t code = 0, t = 0, q_cnt = 0;
      if (item < n_items) {
        load_q(cur);
        load_k(cur, 0);
        load_v(cur, 0);
      }
      int j = 0;
      while (item < n_items && !code) {
        const uint32_t ph = t & 1;
        // the step after this one: next key tile of the item, or tile 0 of the next item
        int n_item = item, n_j = j + 1;
        AttnItem nxt = cur;
        if (n_j >= cur.n_kv) {
          n_j = 0;
          n_item = item + gridDim.x;
          while (n_item < n_items && (nxt = attn_item(p, n_item, q_tiles)).n_kv == 0) n_item += gridDim.x;
        }
        const bool has_next = n_item < n_items;
        if (j == 0) {
          if (!mbar_wait(&bar_q, q_cnt & 1, abort_flag)) { code = 0x51000000u; break; }
          ++q_cnt;
        }
        // S overwrites the columns that held P and O of the previous step: the softmax
        // threads must have read that O (the P.V that read P has completed by then)
        if (t > 0 && !mbar_wait(&bar_o_read, ph ^ 1, abort_flag)) { code = 0x57000000u | (t & 0xffff); break; }
        if (!mbar_wait(&bar_k, ph, abort_flag)) { code = 0x53000000u | (t & 0xffff); break; }
        tc_fence_after();
        {
          const uint64_t a_desc = make_smem_desc_sw128(q_addr, 16, 1024);
          const uint64_t b_desc = make_smem_desc_sw128(k_addr, 16, 1024);
#pragma unroll
          for (int k = 0; k < D / 16; ++k)
            umma_f16_ss(tmem_base + S_COL, a_desc + 2 * k, b_desc + 2 * k, idesc_s, k != 0);
        }
        umma_commit(&bar_s_full);
        if (!mbar_wait(&bar_s_full, ph, abort_flag)) { code = 0x54000000u | (t & 0xffff); break; }
        if (has_next) {
          // K (and, when this was the item's last tile, Q) are free: prefetch the next step's
          if (n_j == 0) load_q(nxt);
          load_k(nxt, n_j);
        }
        if (!mbar_wait(&bar_p_ready, ph, abort_flag)) { code = 0x55000000u | (t & 0xffff); break; }
        if (!mbar_wait(&bar_v, ph, abort_flag)) { code = 0x56000000u | (t & 0xffff); break; }
        tc_fence_after();
        {
#pragma unroll
          for (int k = 0; k < BKV / 16; ++k) {
            // A: P in tensor memory, 16 keys = 8 columns (two 16-bit values per column).
            // B: V as loaded (key rows of 128 bytes): 16 keys = 2048 bytes further.
            const uint64_t b_desc = make_smem_desc_sw128(v_addr + k * 2048, 1024, 1024);
            umma_f16_ts(tmem_base + O_COL, tmem_base + P_COL + k * 8, b_desc, idesc_o, k != 0);
          }
        }
        umma_commit(&bar_o_full);
        if (has_next) {
          // V is free once this P.V has been computed
          if (!mbar_wait(&bar_o_full, ph, abort_flag)) { code = 0x52000000u | (t & 0xffff); break; }
          load_v(nxt, n_j);
        }
        ++t;
        item = n_item;
        j = n_j;
        cur = nxt;
      }
      if (code) atomicCAS(p.err, 0u, code);
    }
  } else {
    // ------------------------------ softmax + output ------------------------------
    const int r = threadIdx.x;  // query row inside the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    uint32_t t = 0;  // key tiles processed so far by this CTA (same count as the control thread)
    bool ok = true;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const AttnItem it = attn_item(p, item, q_tiles);
      const int q_local = it.q0 + r;  // query index inside the sequence
      float o_acc[D];
#pragma unroll
      for (int e = 0; e < D; ++e) o_acc[e] = 0.f;
      float m_run = -INFINITY, l_run = 0.f;
      for (int j = 0; j < it.n_kv && ok; ++j, ++t) {
        const uint32_t ph = t & 1;
        if (!mbar_wait(&bar_s_full, ph, abort_flag)) {
          atomicCAS(p.err, 0u, 0x61000000u | (t & 0xffff));
          ok = false;
          break;
        }
        tc_fence_after();
        // columns (keys) this row may attend to inside the tile: [0, ncol)
        int ncol = it.kv_end - j * BKV;
        if (p.causal) ncol = min(ncol, q_local + 1 - j * BKV);
        ncol = max(min(ncol, BKV), 0);
        // every row of this warp sees the whole tile: no per-element masking
        const bool full_tile = __all_sync(0xffffffffu, ncol == BKV);
        // pass 1: row maximum
        float m_tile = -INFINITY;
        if (full_tile) {
          // 16 columns at a time, the next load in flight while the current piece is reduced
          uint32_t sa[16], sb[16];
          const uint32_t s_addr = tmem_base + lane_addr + S_COL;
          tmem_ld_32x16(s_addr, sa);
#pragma unroll
          for (int c = 0; c < BKV / 16; c += 2) {
            tmem_ld_wait_regs(sa);
            tmem_ld_32x16(s_addr + (c + 1) * 16, sb);
#pragma unroll
            for (int i = 0; i < 16; ++i) m_tile = fmaxf(m_tile, __uint_as_float(sa[i]));
            tmem_ld_wait_regs(sb);
            if (c + 2 < BKV / 16) tmem_ld_32x16(s_addr + (c + 2) * 16, sa);
#pragma unroll
            for (int i = 0; i < 16; ++i) m_tile = fmaxf(m_tile, __uint_as_float(sb[i]));
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < BKV / 32; ++c) {
            uint32_t s[32];
            tmem_ld_32x32(tmem_base + lane_addr + S_COL + c * 32, s);
            tmem_ld_wait_regs(s);
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i < ncol) m_tile = fmaxf(m_tile, __uint_as_float(s[i]));
          }
        }
        const float m_new = fmaxf(m_run, m_tile);
        // rows with no visible key yet keep m = -inf; use 0 as the reference point then
        const float m_ref = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = m_run == -INFINITY ? 0.f : ex2_fast((m_run - m_ref) * p.scale_log2e);
        // pass 2: P = exp2((s - m) * c) and its row sum; the 16-bit P of keys [32c, 32c+32)
        // goes to columns [16c, 16c+16), over S columns this thread has already consumed
        float l_tile = 0.f;
        const float mc = m_ref * p.scale_log2e;
        if (full_tile) {
          // the same pipelining; two 16-column pieces of S make one 16-register piece of P
          uint32_t sa[16], sb[16];
          const uint32_t s_addr = tmem_base + lane_addr + S_COL;
          tmem_ld_32x16(s_addr, sa);
#pragma unroll
          for (int c = 0; c < BKV / 16; c += 2) {
            uint32_t packed[16];
            tmem_ld_wait_regs(sa);
            tmem_ld_32x16(s_addr + (c + 1) * 16, sb);
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              const float p0 = ex2_fast(fmaf(__uint_as_float(sa[i]), p.scale_log2e, -mc));
              const float p1 = ex2_fast(fmaf(__uint_as_float(sa[i + 1]), p.scale_log2e, -mc));
              l_tile += p0 + p1;
              packed[i >> 1] = pack16<T16>(p0, p1);
            }
            tmem_ld_wait_regs(sb);
            // the P piece below overwrites S columns [8c, 8c + 16): all of them have been read
            // (this thread is past column 16c + 32), so the next S load may start first
            if (c + 2 < BKV / 16) tmem_ld_32x16(s_addr + (c + 2) * 16, sa);
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              const float p0 = ex2_fast(fmaf(__uint_as_float(sb[i]), p.scale_log2e, -mc));
              const float p1 = ex2_fast(fmaf(__uint_as_float(sb[i + 1]), p.scale_log2e, -mc));
              l_tile += p0 + p1;
              packed[8 + (i >> 1)] = pack16<T16>(p0, p1);
            }
            tmem_st_32x16(tmem_base + lane_addr + P_COL + (c / 2) * 16, packed);
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < BKV / 32; ++c) {
            uint32_t s[32];
            tmem_ld_32x32(tmem_base + lane_addr + S_COL + c * 32, s);
            tmem_ld_wait_regs(s);
            uint32_t packed[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float p0 = 0.f, p1 = 0.f;
              if (c * 32 + i < ncol) p0 = ex2_fast(fmaf(__uint_as_float(s[i]), p.scale_log2e, -mc));
              if (c * 32 + i + 1 < ncol) p1 = ex2_fast(fmaf(__uint_as_float(s[i + 1]), p.scale_log2e, -mc));
              l_tile += p0 + p1;
              packed[i >> 1] = pack16<T16>(p0, p1);
            }
            tmem_st_32x16(tmem_base + lane_addr + P_COL + c * 16, packed);
          }
        }
        l_run = fmaf(l_run, alpha, l_tile);
        m_run = m_new;
        // P is in tensor memory and every S column of this tile has been read
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&bar_p_ready);
        // O_t = P.V of this tile: fold it into the running output, then hand the columns back
        if (!mbar_wait(&bar_o_full, ph, abort_flag)) {
          atomicCAS(p.err, 0u, 0x62000000u | (t & 0xffff));
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(tmem_base + lane_addr + O_COL + c * 32, o);
          tmem_ld_wait_regs(o);
#pragma unroll
          for (int i = 0; i < 32; ++i)
            o_acc[c * 32 + i] = fmaf(o_acc[c * 32 + i], alpha, __uint_as_float(o[i]));
        }
        tc_fence_before();
        mbar_arrive(&bar_o_read);
      }
      if (ok && q_local < p.seq) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        T16 *dst = static_cast<T16 *>(p.out) + static_cast<size_t>(it.row_base + q_local) * hd + it.head * D;
#pragma unroll
        for (int g = 0; g < D / 8; ++g) {
          uint4 o;
          o.x = pack16<T16>(o_acc[8 * g + 0] * inv, o_acc[8 * g + 1] * inv);
          o.y = pack16<T16>(o_acc[8 * g + 2] * inv, o_acc[8 * g + 3] * inv);
          o.z = pack16<T16>(o_acc[8 * g + 4] * inv, o_acc[8 * g + 5] * inv);
          o.w = pack16<T16>(o_acc[8 * g + 6] * inv, o_acc[8 * g + 7] * inv);
          reinterpret_cast<uint4 *>(dst)[g] = o;
        }
      }
    }
  }

  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 4) tmem_dealloc(tmem_base, TMEM_COLS);
}

bool encode_tmap_2d(CUtensorMap *map, const void *base, int32_t dtype, uint64_t inner, uint64_t outer,
                    uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);

}  // namespace mdc

using namespace mdc;

MDC_API void mgpuAttention(const void *qkv, const int32_t *seq_lens, void *out, int64_t batch,
                           int64_t seq_len, int64_t heads, int64_t head_dim, bool causal,
                           int32_t dtype, void *stream) {
  if (batch <= 0 || seq_len <= 0 || heads <= 0) return;
  const DeviceInfo &di = device_info();
  if (!di.ok) return;
  if (head_dim != attn::D) { fail("mgpuAttention: head_dim must be 64"); return; }
  if (!dtype_is16(dtype)) { fail("mgpuAttention: dtype must be F16 or BF16"); return; }
  if ((reinterpret_cast<uintptr_t>(qkv) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u)) {
    fail("mgpuAttention: buffers must be 16-byte aligned");
    return;
  }
  const int64_t tokens = batch * seq_len;
  const int64_t q_tiles = (seq_len + attn::BQ - 1) / attn::BQ;
  if (tokens > 0x7fffffff || heads > 65535 || batch > 65535) { fail("mgpuAttention: shape too large"); return; }
  uint32_t *err = device_error_slot();
  if (!err) return;
  CUtensorMap tm;
  const uint64_t row_elems = static_cast<uint64_t>(3 * heads * attn::D);
  if (!encode_tmap_2d(&tm, qkv, dtype, row_elems, static_cast<uint64_t>(tokens), row_elems * 2, attn::D, 128))
    return;
  AttnParams p;
  p.seq_lens = seq_lens;
  p.out = out;
  p.batch = static_cast<int>(batch);
  p.seq = static_cast<int>(seq_len);
  p.heads = static_cast<int>(heads);
  p.causal = causal ? 1 : 0;
  p.scale_log2e = 1.4426950408889634f / sqrtf(static_cast<float>(attn::D));
  p.err = err;
  const int64_t n_items = q_tiles * heads * batch;
  if (n_items > 0x7fffffff) { fail("mgpuAttention: shape too large"); return; }
  // persistent CTAs, three per SM (49 KiB of shared memory and 128 TMEM columns each)
  const int64_t slots = static_cast<int64_t>(di.sms) * attn::CTAS_PER_SM;
  dim3 grid(static_cast<unsigned>(n_items < slots ? n_items : slots));
  cudaStream_t s = as_stream(stream);
  ProfileScope prof(kCatAttention, s);
  if (dtype == MGPU_DTYPE_F16) {
    auto kern = attention_tcgen05_kernel<__half>;
    static bool set_on[64] = {false};  // the attribute is per device
    bool &set = set_on[(di.device >= 0 && di.device < 64) ? di.device : 0];
    if (!set) {
      if (!check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(attn::SMEM_BYTES)), "cudaFuncSetAttribute(attention)"))
        return;
      set = true;
    }
    check_cuda(launch_chain(kern, grid, dim3(attn::THREADS), attn::SMEM_BYTES, s, 1, tm, p), "launch attention");
  } else {
    auto kern = attention_tcgen05_kernel<__nv_bfloat16>;
    static bool set_on[64] = {false};  // the attribute is per device
    bool &set = set_on[(di.device >= 0 && di.device < 64) ? di.device : 0];
    if (!set) {
      if (!check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(attn::SMEM_BYTES)), "cudaFuncSetAttribute(attention)"))
        return;
      set = true;
    }
    check_cuda(launch_chain(kern, grid, dim3(attn::THREADS), attn::SMEM_BYTES, s, 1, tm, p), "launch attention");
  }
  launched("attention_tcgen05_kernel");
}
