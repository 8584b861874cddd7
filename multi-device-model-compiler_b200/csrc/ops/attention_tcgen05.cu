// Fused multi-head attention for sm_100a, head_dim 64 or 128, fp16 / bf16:
//   out = softmax(Q.K^T / sqrt(d) + mask) . V        per (batch, head)
// on the packed QKV Gemm output [tokens, 3, heads, head_dim].  Replaces the vendored
// FusedMHARunnerFP16v2 (precompiled sm_70..sm_89 cubins, built for 8 heads x 128,
// lib/Kernels/GPU/LLM.cu:18-19) that the reference layer calls at lib/Kernels/GPU/LLM.cu:79-81;
// masks: key padding from per-sequence lengths and, optionally, causal.
//
// One persistent CTA walks work items (128 queries of one (sequence, head)) and, inside an
// item, the keys in tiles of 128 (flash-style online softmax; fully masked tiles are skipped).
// The key tiles of all its items form one sequence of steps t = 0, 1, ...  Six warps:
//   warp 5, one thread   TMA producer: Q tile per item, K and V tile per step, 128-byte
//                        swizzled, completion on mbarriers (two stages each at head_dim 64).
//   warp 4, one thread   MMA issuer.  Per step two tcgen05.mma groups:
//                          S = Q.K^T   (M=128, N=128, K=head_dim) -> TMEM columns [0,128)
//                          O += P.V    (M=128, N=head_dim, K=128)  -> one of two output buffers behind S
//                        P (16-bit, two keys per 32-bit column) is written by the softmax
//                        threads over the S columns [0,64) and is the A operand of the second
//                        MMA straight from tensor memory; V is used as it lies in memory (keys x
//                        head_dim, an MN-major B operand), so there is no transpose pass.  The
//                        output accumulates in tensor memory across the key tiles of an item.
//   warps 0-3            one thread per query row.  Per step ONE read of the row's 128 scores
//                        into registers (four tcgen05.ld in flight, one wait), row maximum,
//                        P = exp2(..) and row sum from the same registers, P stored back with
//                        tcgen05.st.  The running maximum is only raised when the new one exceeds
//                        it by more than 2^8 (in the exponent's units); then, and only then, the
//                        accumulated O in tensor memory is rescaled (ld, multiply, st).  Results are
//                        exact either way: P and the row sum use the same reference point, and the
//                        final division cancels it.  An item's output is written one step late:
//                        consecutive items alternate between two O buffers in tensor memory, and
//                        when the scores of the next step arrive (the MMAs complete in order, so
//                        the item's last P.V has completed too) the thread reads its O row,
//                        divides by the row sum and stages it in shared memory, from where each
//                        warp writes its 32 rows with one TMA store (whole lines, clipped at the
//                        end of the sequence).
// head_dim 64: 256 TMEM columns and 97 KiB of shared memory per CTA, two CTAs per SM, which
// fill each other's waits (one CTA's MMA and loads run under the other's softmax).
// head_dim 128: 384 columns (512 allocated), 193 KiB, one CTA per SM.
// The tensor map is three-dimensional (column, position in sequence, sequence), so tile rows
// past the end of a sequence are zero-filled by TMA and never read from the next sequence.
// Rows of padded positions inside a sequence (seq_lens[b] <= position < seq_len) are loaded as
// they are: their scores are masked, but they must hold finite values.  Every wait is bounded.
#include <cstdlib>
#include <type_traits>

#include "ops_common.h"
#include "ptx_sm100.cuh"

namespace mdc {

namespace attn {
constexpr int BQ = 128, BKV = 128;
constexpr int THREADS = 192;
constexpr int BLOCK_BYTES = 128 * 64 * 2;  // one 128-row x 64-column swizzled block: 16 KiB
constexpr int S_COL = 0, O_COL = 128;      // two O buffers of head_dim columns follow S
constexpr float kRescaleThreshold = 8.f;   // raise the running maximum only beyond 2^8
template <int HD>
struct Cfg {
  static constexpr int BLOCKS = HD / 64;                   // 64-column blocks per tile
  static constexpr int TILE_BYTES = BLOCKS * BLOCK_BYTES;  // 16 / 32 KiB
  static constexpr int Q_STAGES = 1;
  static constexpr int KV_STAGES = 2;
  static constexpr int TMEM_COLS = HD == 64 ? 256 : 512;
  static constexpr int CTAS_PER_SM = HD == 64 ? 2 : 1;
  static constexpr int OUT_WARP_BYTES = BLOCKS * 4096;     // staged output of one warp: 32 rows
  static constexpr size_t SMEM_BYTES =
      static_cast<size_t>(Q_STAGES + 2 * KV_STAGES) * TILE_BYTES + 4 * OUT_WARP_BYTES + 1024;
};
}  // namespace attn

struct AttnParams {
  const int32_t *seq_lens;  // [batch] or nullptr
  void *out;                // [batch*seq, heads*head_dim]
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

// One unit of work: 128 queries of one (sequence, head).  Decoded identically by all three
// roles, so they walk the same sequence of key tiles.
struct AttnItem {
  int q0, head, b, kv_end, n_kv;
};
__device__ __forceinline__ AttnItem attn_item(const AttnParams &p, int item, int q_tiles) {
  AttnItem it;
  const int qt = item % q_tiles;
  const int rest = item / q_tiles;
  it.head = rest % p.heads;
  it.b = rest / p.heads;
  it.q0 = qt * attn::BQ;
  const int len = p.seq_lens ? min(max(p.seq_lens[it.b], 0), p.seq) : p.seq;
  it.kv_end = p.causal ? min(len, it.q0 + attn::BQ) : len;  // keys this query tile can see: [0, kv_end)
  // a tile whose queries are all padding (q0 >= len) does no work: its rows are written as zeros
  it.n_kv = it.q0 < len ? (it.kv_end + attn::BKV - 1) / attn::BKV : 0;
  return it;
}

__device__ __forceinline__ float ex2_fast(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

template <typename T16, int HD>
__global__ void __launch_bounds__(attn::THREADS, attn::Cfg<HD>::CTAS_PER_SM)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_qkv,
                         const __grid_constant__ CUtensorMap tmap_out, const AttnParams p) {
  using namespace attn;
  using namespace ptx;
  using C = Cfg<HD>;
  constexpr int TILE_BYTES = C::TILE_BYTES, QS = C::Q_STAGES, KS = C::KV_STAGES;
  extern __shared__ uint8_t smem_dyn[];
  __shared__ uint64_t q_full[QS], q_empty[QS], k_full[KS], k_empty[KS], v_full[KS], v_empty[KS];
  __shared__ uint64_t s_full, p_ready, all_done;
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t abort_flag_s;
  volatile uint32_t *abort_flag = &abort_flag_s;

  uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
  uint8_t *sQ = tiles, *sK = tiles + QS * TILE_BYTES, *sV = sK + KS * TILE_BYTES;
  uint8_t *sOut = sV + KS * TILE_BYTES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tiles = (p.seq + BQ - 1) / BQ;
  const int n_items = q_tiles * p.heads * p.batch;
  const int hd = p.heads * HD;

  if (threadIdx.x == 0) {
    abort_flag_s = 0;
    tma_prefetch_desc(&tmap_qkv);
    for (int i = 0; i < QS; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    for (int i = 0; i < KS; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    mbar_init(&s_full, 1);
    mbar_init(&p_ready, 128);
    mbar_init(&all_done, 1);
    mbar_init_fence();
  }
  if (warp == 4) {
    tmem_alloc(&tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  pdl_launch_dependents();  // after this CTA holds its tensor memory (see the Gemm kernel)
  pdl_wait();  // set-up above overlaps the previous kernel's tail; QKV is read below

  if (warp == 5) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t t = 0, qn = 0, code = 0;
      for (int item = blockIdx.x; item < n_items && !code; item += gridDim.x) {
        const AttnItem it = attn_item(p, item, q_tiles);
        if (it.n_kv == 0) continue;
        const uint32_t qs = qn % QS;
        if (!mbar_wait(&q_empty[qs], ((qn / QS) & 1) ^ 1, abort_flag)) { code = 0x71000000u; break; }
        mbar_arrive_expect_tx(&q_full[qs], TILE_BYTES);
#pragma unroll
        for (int blk = 0; blk < C::BLOCKS; ++blk)
          tma_load_3d(sQ + qs * TILE_BYTES + blk * BLOCK_BYTES, &tmap_qkv, &q_full[qs],
                      it.head * HD + blk * 64, it.q0, it.b);
        ++qn;
        for (int j = 0; j < it.n_kv; ++j, ++t) {
          const uint32_t st = t % KS, ph = ((t / KS) & 1) ^ 1;
          if (!mbar_wait(&k_empty[st], ph, abort_flag)) { code = 0x72000000u | (t & 0xffff); break; }
          mbar_arrive_expect_tx(&k_full[st], TILE_BYTES);
#pragma unroll
          for (int blk = 0; blk < C::BLOCKS; ++blk)
            tma_load_3d(sK + st * TILE_BYTES + blk * BLOCK_BYTES, &tmap_qkv, &k_full[st],
                        hd + it.head * HD + blk * 64, j * BKV, it.b);
          if (!mbar_wait(&v_empty[st], ph, abort_flag)) { code = 0x73000000u | (t & 0xffff); break; }
          mbar_arrive_expect_tx(&v_full[st], TILE_BYTES);
#pragma unroll
          for (int blk = 0; blk < C::BLOCKS; ++blk)
            tma_load_3d(sV + st * TILE_BYTES + blk * BLOCK_BYTES, &tmap_qkv, &v_full[st],
                        2 * hd + it.head * HD + blk * 64, j * BKV, it.b);
        }
      }
      if (code) atomicCAS(p.err, 0u, code);
    }
  } else if (warp == 4) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr bool kBf16 = std::is_same<T16, __nv_bfloat16>::value;
      constexpr uint32_t idesc_s = make_idesc_f16(BQ, BKV, kBf16, false, false);
      constexpr uint32_t idesc_o = make_idesc_f16(BQ, 64, kBf16, false, true);  // V is MN-major
      const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      uint32_t t = 0, qn = 0, code = 0;
      for (int item = blockIdx.x; item < n_items && !code; item += gridDim.x) {
        const AttnItem it = attn_item(p, item, q_tiles);
        if (it.n_kv == 0) continue;
        const uint32_t qs = qn % QS;
        if (!mbar_wait(&q_full[qs], (qn / QS) & 1, abort_flag)) { code = 0x51000000u; break; }
        for (int j = 0; j < it.n_kv; ++j, ++t) {
          const uint32_t st = t % KS, ph = (t / KS) & 1;
          // S = Q.K^T.  It overwrites the scores / P of the previous step, which the P.V issued
          // just before has finished reading by the time this executes (one in-order pipe).
          if (!mbar_wait(&k_full[st], ph, abort_flag)) { code = 0x53000000u | (t & 0xffff); break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            const uint64_t a_desc = make_smem_desc_sw128(q_addr + qs * TILE_BYTES + (kk / 4) * BLOCK_BYTES, 16, 1024);
            const uint64_t b_desc = make_smem_desc_sw128(k_addr + st * TILE_BYTES + (kk / 4) * BLOCK_BYTES, 16, 1024);
            umma_f16_ss(tmem_base + S_COL, a_desc + 2 * (kk % 4), b_desc + 2 * (kk % 4), idesc_s, kk != 0);
          }
          umma_commit(&s_full);
          umma_commit(&k_empty[st]);
          if (j == it.n_kv - 1) umma_commit(&q_empty[qs]);
          // O (+)= P.V, one N = 64 MMA group per 64 output columns
          if (!mbar_wait(&p_ready, t & 1, abort_flag)) { code = 0x55000000u | (t & 0xffff); break; }
          if (!mbar_wait(&v_full[st], ph, abort_flag)) { code = 0x56000000u | (t & 0xffff); break; }
          tc_fence_after();
#pragma unroll
          for (int nb = 0; nb < C::BLOCKS; ++nb) {
#pragma unroll
            for (int k = 0; k < BKV / 16; ++k) {
              // A: P in tensor memory, 16 keys = 8 columns (two 16-bit values per column).
              // B: V as loaded (key rows of 128 bytes): 16 keys = 2048 bytes further.
              const uint64_t b_desc = make_smem_desc_sw128(v_addr + st * TILE_BYTES + nb * BLOCK_BYTES + k * 2048, 1024, 1024);
              umma_f16_ts(tmem_base + O_COL + (qn & 1) * HD + nb * 64, tmem_base + S_COL + k * 8, b_desc, idesc_o, (j | k) != 0);
            }
          }
          umma_commit(&v_empty[st]);
        }
        ++qn;
      }
      umma_commit(&all_done);  // everything issued above has completed
      if (code) atomicCAS(p.err, 0u, code);
    }
  } else {
    // ------------------------------ softmax + output ------------------------------
    const int r = threadIdx.x;  // query row inside the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_addr + S_COL;
    uint8_t *my_out = sOut + warp * C::OUT_WARP_BYTES;
    uint32_t t = 0;   // key tiles processed so far by this CTA (same count as the other roles)
    uint32_t qn = 0;  // items with at least one key tile started so far
    bool ok = true;
    // the finished item whose output still sits in its O buffer
    bool pending = false;
    uint32_t pend_buf = 0;
    int pend_x = 0, pend_y = 0, pend_z = 0;
    float pend_inv = 0.f;

    // O / l of the pending item -> shared memory (swizzled 128-byte rows) -> one TMA store
    // per 64 columns; rows past the end of the sequence are clipped by the tensor map
    auto write_pending = [&]() {
      const uint32_t o_addr = tmem_base + lane_addr + O_COL + pend_buf * HD;
      if (lane == 0) tma_store_wait_read<0>();  // the previous store has left the staging buffer
      __syncwarp();
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(o_addr + c * 32, o);
        tmem_ld_wait_regs(o);
        // 32 columns = 64 bytes = four 16-byte pieces of this row's 128-byte line
        uint8_t *row = my_out + (c / 2) * 4096 + lane * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 v;
          v.x = pack16<T16>(__uint_as_float(o[8 * g + 0]) * pend_inv, __uint_as_float(o[8 * g + 1]) * pend_inv);
          v.y = pack16<T16>(__uint_as_float(o[8 * g + 2]) * pend_inv, __uint_as_float(o[8 * g + 3]) * pend_inv);
          v.z = pack16<T16>(__uint_as_float(o[8 * g + 4]) * pend_inv, __uint_as_float(o[8 * g + 5]) * pend_inv);
          v.w = pack16<T16>(__uint_as_float(o[8 * g + 6]) * pend_inv, __uint_as_float(o[8 * g + 7]) * pend_inv);
          const int piece = ((c & 1) * 4 + g) ^ (lane & 7);
          *reinterpret_cast<uint4 *>(row + (piece << 4)) = v;
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
#pragma unroll
        for (int blk = 0; blk < C::BLOCKS; ++blk)
          tma_store_3d(&tmap_out, my_out + blk * 4096, pend_x + blk * 64, pend_y + warp * 32, pend_z);
        tma_store_commit();
      }
      pending = false;
    };

    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const AttnItem it = attn_item(p, item, q_tiles);
      const int q_local = it.q0 + r;  // query index inside the sequence
      if (it.n_kv == 0) {
        // no visible key (zero-length sequence): the output rows are zeros
        if (q_local < p.seq) {
          T16 *dst = static_cast<T16 *>(p.out) + (static_cast<size_t>(it.b) * p.seq + q_local) * hd + it.head * HD;
#pragma unroll
          for (int g = 0; g < HD / 8; ++g) reinterpret_cast<uint4 *>(dst)[g] = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      const uint32_t o_addr = tmem_base + lane_addr + O_COL + (qn & 1) * HD;
      // m_run is the reference point of the exponent (in score units), l_run the row sum
      float m_run = -INFINITY, l_run = 0.f;
      for (int j = 0; j < it.n_kv && ok; ++j, ++t) {
        if (!mbar_wait(&s_full, t & 1, abort_flag)) {
          atomicCAS(p.err, 0u, 0x61000000u | (t & 0xffff));
          ok = false;
          break;
        }
        tc_fence_after();
        // The MMAs complete in order: with these scores the previous item's last P.V has
        // completed as well, so its output can leave now.
        if (pending) write_pending();
        // the whole row of scores: four loads in flight, one wait
        uint32_t s0[32], s1[32], s2[32], s3[32];
        tmem_ld_32x32(s_addr, s0);
        tmem_ld_32x32(s_addr + 32, s1);
        tmem_ld_32x32(s_addr + 64, s2);
        tmem_ld_32x32(s_addr + 96, s3);
        // columns (keys) this row may attend to inside the tile: [0, ncol)
        int ncol = it.kv_end - j * BKV;
        if (p.causal) ncol = min(ncol, q_local + 1 - j * BKV);
        ncol = max(min(ncol, BKV), 0);
        // every row of this warp sees the whole tile: no per-element masking
        const bool full_tile = __all_sync(0xffffffffu, ncol == BKV);
        tmem_ld_wait_regs(s0);
        tmem_ld_wait_regs(s1);
        tmem_ld_wait_regs(s2);
        tmem_ld_wait_regs(s3);
        if (!full_tile) {
          // masked scores become -inf: they drop out of the maximum and give P = 0
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (i >= ncol) s0[i] = 0xff800000u;
            if (32 + i >= ncol) s1[i] = 0xff800000u;
            if (64 + i >= ncol) s2[i] = 0xff800000u;
            if (96 + i >= ncol) s3[i] = 0xff800000u;
          }
        }
        float m_tile = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          m_tile = fmaxf(m_tile, fmaxf(__uint_as_float(s0[i]), __uint_as_float(s1[i])));
          m_tile = fmaxf(m_tile, fmaxf(__uint_as_float(s2[i]), __uint_as_float(s3[i])));
        }
        // Raise the reference point only when the new maximum exceeds it by more than the
        // threshold (always on the first tile with a visible key).
        const bool raise = m_tile > m_run && (m_run == -INFINITY || (m_tile - m_run) * p.scale_log2e > kRescaleThreshold);
        float alpha = 1.f;
        if (raise) {
          alpha = m_run == -INFINITY ? 0.f : ex2_fast((m_run - m_tile) * p.scale_log2e);
          m_run = m_tile;
          l_run *= alpha;
        }
        // the rescaling uses warp-wide tensor-memory instructions: decided per warp
        if (j > 0 && __any_sync(0xffffffffu, raise)) {
          // O holds the sum over the earlier tiles (their P.V has completed: S of this step
          // was issued after it on the same in-order pipe): bring it to the new reference point
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(o_addr + c * 32, o);
            tmem_ld_wait_regs(o);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(o_addr + c * 32, o);
          }
        }
        // rows with no visible key yet keep m = -inf; use 0 as the reference point then
        const float mc = (m_run == -INFINITY ? 0.f : m_run) * p.scale_log2e;
        float l_a = 0.f, l_b = 0.f;
        // P = exp2((s - m) * c), 16-bit, two keys per column: keys [32q, 32q+32) -> columns [16q, 16q+16)
#define MDC_ATTN_P_PIECE(SREG, Q)                                                               \
  {                                                                                             \
    uint32_t packed[16];                                                                        \
    _Pragma("unroll") for (int i = 0; i < 32; i += 2) {                                         \
      const float p0 = ex2_fast(fmaf(__uint_as_float(SREG[i]), p.scale_log2e, -mc));            \
      const float p1 = ex2_fast(fmaf(__uint_as_float(SREG[i + 1]), p.scale_log2e, -mc));        \
      l_a += p0;                                                                                \
      l_b += p1;                                                                                \
      packed[i >> 1] = pack16<T16>(p0, p1);                                                     \
    }                                                                                           \
    tmem_st_32x16(s_addr + (Q) * 16, packed);                                                   \
  }
        MDC_ATTN_P_PIECE(s0, 0)
        MDC_ATTN_P_PIECE(s1, 1)
        MDC_ATTN_P_PIECE(s2, 2)
        MDC_ATTN_P_PIECE(s3, 3)
#undef MDC_ATTN_P_PIECE
        l_run += l_a + l_b;
        // P (and a rescaled O) are in tensor memory and every S column of this tile has been read
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&p_ready);
      }
      if (!ok) break;
      pending = true;
      pend_buf = qn & 1;
      pend_x = it.head * HD;
      pend_y = it.q0;
      pend_z = it.b;
      pend_inv = l_run > 0.f ? 1.f / l_run : 0.f;
      ++qn;
    }
    if (ok && pending) {
      if (!mbar_wait(&all_done, 0, abort_flag)) {
        atomicCAS(p.err, 0u, 0x62000000u);
      } else {
        tc_fence_after();
        write_pending();
      }
    }
    if (lane == 0) tma_store_wait<0>();  // all staged output has left shared memory
  }

  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 4) tmem_dealloc(tmem_base, C::TMEM_COLS);
}


// ------------------------------------------------------------------------------------------
// head_dim 64.  Same work decomposition, different use of the SM: a CTA keeps ONE score
// buffer (S in TMEM columns [0,128), then P in [0,64) and the partial product O_t in [64,128))
// and folds O_t into output registers after every key tile, so it needs only 128 TMEM columns
// and 65 KiB of shared memory and THREE CTAs share an SM, overlapping each other's load / MMA /
// softmax phases.  Measured at 12 heads x 64 this beats the general kernel above run at the
// same head size (40 vs 63 us for 256 sequences of 128 tokens, 35 vs 56 us for 32 padded
// sequences of 384): per key tile a row costs about 1500 cycles of the SM's conversion /
// exponential unit, and what keeps that unit fed is the number of independent rows in flight.
//   warp 4, one thread   TMA loads of the Q / K / V tiles and both MMA groups per key tile;
//                        the loads of the next step are issued while the current one is in
//                        its softmax (K after S has been computed, V after P.V has).
//   warps 0-3            one thread per query row: two passes over the scores in pieces of 16
//                        columns (maximum; then P and the row sum), O_t read back and
//                        accumulated in registers with the usual rescaling; the item's rows
//                        leave through shared memory and one TMA store per warp.
// ------------------------------------------------------------------------------------------
namespace attn64 {
constexpr int BQ = 128, BKV = 128, D = 64;
constexpr int TILE_BYTES = 128 * D * 2;  // 16 KiB: one 128 x 64 16-bit tile
constexpr int THREADS = 160;
constexpr int TMEM_COLS = 128;
constexpr int S_COL = 0, P_COL = 0, O_COL = 64;
constexpr int CTAS_PER_SM = 3;
constexpr size_t SMEM_BYTES = 3 * TILE_BYTES + 4 * 4096 + 1024;
}  // namespace attn64

struct AttnItem64 {
  int q0, head, b, kv_end, n_kv;
};
__device__ __forceinline__ AttnItem64 attn_item64(const AttnParams &p, int item, int q_tiles) {
  AttnItem64 it;
  const int qt = item % q_tiles;
  const int rest = item / q_tiles;
  it.head = rest % p.heads;
  it.b = rest / p.heads;
  it.q0 = qt * attn64::BQ;
  const int len = p.seq_lens ? min(max(p.seq_lens[it.b], 0), p.seq) : p.seq;
  it.kv_end = p.causal ? min(len, it.q0 + attn64::BQ) : len;  // keys this query tile can see: [0, kv_end)
  // a tile whose queries are all padding (q0 >= len) does no work: its rows are written as zeros
  it.n_kv = it.q0 < len ? (it.kv_end + attn64::BKV - 1) / attn64::BKV : 0;
  return it;
}

// Persistent: each CTA walks work items item = blockIdx.x, + gridDim.x, ...; the key tiles of
// all its items form one sequence of steps t = 0, 1, ..., and every barrier completes once
// per step (parity t & 1), so loads for step t+1 (of the same or of the next item) are issued
// while step t is still in its softmax: K (and the next item's Q) as soon as S = Q.K^T of
// step t has been computed, V as soon as P.V of step t has.
template <typename T16>
__global__ void __launch_bounds__(attn64::THREADS, attn64::CTAS_PER_SM)
attention_d64_kernel(const __grid_constant__ CUtensorMap tmap_qkv,
                     const __grid_constant__ CUtensorMap tmap_out, const AttnParams p) {
  using namespace attn64;
  using namespace ptx;
  extern __shared__ uint8_t smem_dyn[];
  __shared__ uint64_t bar_q, bar_k, bar_v, bar_s_full, bar_p_ready, bar_o_full, bar_o_read;
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t abort_flag_s;
  volatile uint32_t *abort_flag = &abort_flag_s;

  uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
  uint8_t *sQ = tiles, *sK = tiles + TILE_BYTES, *sV = tiles + 2 * TILE_BYTES;
  uint8_t *sOut = tiles + 3 * TILE_BYTES;  // 4 warps x 32 rows x 128 bytes of staged output

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
      auto load_q = [&](const AttnItem64 &it) {
        mbar_arrive_expect_tx(&bar_q, TILE_BYTES);
        tma_load_3d(sQ, &tmap_qkv, &bar_q, it.head * D, it.q0, it.b);
      };
      auto load_k = [&](const AttnItem64 &it, int j) {
        mbar_arrive_expect_tx(&bar_k, TILE_BYTES);
        tma_load_3d(sK, &tmap_qkv, &bar_k, hd + it.head * D, j * BKV, it.b);
      };
      auto load_v = [&](const AttnItem64 &it, int j) {
        mbar_arrive_expect_tx(&bar_v, TILE_BYTES);
        tma_load_3d(sV, &tmap_qkv, &bar_v, 2 * hd + it.head * D, j * BKV, it.b);
      };
      // first item with at least one visible key
      int item = blockIdx.x;
      AttnItem64 cur{};
      while (item < n_items && (cur = attn_item64(p, item, q_tiles)).n_kv == 0) item += gridDim.x;
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
        AttnItem64 nxt = cur;
        if (n_j >= cur.n_kv) {
          n_j = 0;
          n_item = item + gridDim.x;
          while (n_item < n_items && (nxt = attn_item64(p, n_item, q_tiles)).n_kv == 0) n_item += gridDim.x;
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
      const AttnItem64 it = attn_item64(p, item, q_tiles);
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
      if (ok) {
        // O / l -> shared memory (swizzled 128-byte rows) -> one TMA store of the warp's 32 rows:
        // whole lines, and rows past the end of the sequence are clipped by the tensor map
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        uint8_t *my_out = sOut + warp * 4096;
        if (lane == 0) tma_store_wait_read<0>();  // the previous store has left the staging buffer
        __syncwarp();
#pragma unroll
        for (int g = 0; g < D / 8; ++g) {
          uint4 o;
          o.x = pack16<T16>(o_acc[8 * g + 0] * inv, o_acc[8 * g + 1] * inv);
          o.y = pack16<T16>(o_acc[8 * g + 2] * inv, o_acc[8 * g + 3] * inv);
          o.z = pack16<T16>(o_acc[8 * g + 4] * inv, o_acc[8 * g + 5] * inv);
          o.w = pack16<T16>(o_acc[8 * g + 6] * inv, o_acc[8 * g + 7] * inv);
          *reinterpret_cast<uint4 *>(my_out + lane * 128 + ((g ^ (lane & 7)) << 4)) = o;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_3d(&tmap_out, my_out, it.head * D, it.q0 + warp * 32, it.b);
          tma_store_commit();
        }
      }
    }
    if (lane == 0) tma_store_wait<0>();  // all staged output has left shared memory
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

template <typename T16>
static void launch_attention64(const CUtensorMap &tm, const CUtensorMap &tmo, const AttnParams &p, int64_t n_items,
                               const DeviceInfo &di, cudaStream_t s) {
  auto kern = attention_d64_kernel<T16>;
  static bool set_on[64] = {false};  // the attribute is per device
  bool &set = set_on[(di.device >= 0 && di.device < 64) ? di.device : 0];
  if (!set) {
    if (!check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(attn64::SMEM_BYTES)), "cudaFuncSetAttribute(attention)"))
      return;
    set = true;
  }
  const int64_t slots = static_cast<int64_t>(di.sms) * attn64::CTAS_PER_SM;
  dim3 grid(static_cast<unsigned>(n_items < slots ? n_items : slots));
  check_cuda(launch_chain(kern, grid, dim3(attn64::THREADS), attn64::SMEM_BYTES, s, 1, tm, tmo, p), "launch attention");
}

template <typename T16, int HD>
static void launch_attention(const CUtensorMap &tm, const CUtensorMap &tmo, const AttnParams &p, int64_t n_items, const DeviceInfo &di,
                             cudaStream_t s) {
  using C = attn::Cfg<HD>;
  auto kern = attention_tcgen05_kernel<T16, HD>;
  static bool set_on[64] = {false};  // the attribute is per device
  bool &set = set_on[(di.device >= 0 && di.device < 64) ? di.device : 0];
  if (!set) {
    if (!check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(C::SMEM_BYTES)), "cudaFuncSetAttribute(attention)"))
      return;
    set = true;
  }
  // persistent CTAs: as many as the device holds at once (shared memory and tensor memory)
  const int64_t slots = static_cast<int64_t>(di.sms) * C::CTAS_PER_SM;
  dim3 grid(static_cast<unsigned>(n_items < slots ? n_items : slots));
  check_cuda(launch_chain(kern, grid, dim3(attn::THREADS), C::SMEM_BYTES, s, 1, tm, tmo, p), "launch attention");
}

}  // namespace mdc

using namespace mdc;


MDC_API void mgpuAttention(const void *qkv, const int32_t *seq_lens, void *out, int64_t batch,
                           int64_t seq_len, int64_t heads, int64_t head_dim, bool causal,
                           int32_t dtype, void *stream) {
  if (batch <= 0 || seq_len <= 0 || heads <= 0) return;
  const DeviceInfo &di = device_info();
  if (!di.ok) return;
  if (head_dim != 64 && head_dim != 128) { fail("mgpuAttention: head_dim must be 64 or 128"); return; }
  if (!dtype_is16(dtype)) { fail("mgpuAttention: dtype must be F16 or BF16"); return; }
  if ((reinterpret_cast<uintptr_t>(qkv) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u)) {
    fail("mgpuAttention: buffers must be 16-byte aligned");
    return;
  }
  const int64_t tokens = batch * seq_len;
  const int64_t q_tiles = (seq_len + attn::BQ - 1) / attn::BQ;
  if (tokens > 0x7fffffff || heads > 65535 || batch > 0x7fffffff) { fail("mgpuAttention: shape too large"); return; }
  uint32_t *err = device_error_slot();
  if (!err) return;
  // (column, position, sequence): rows past the end of a sequence are out of bounds for TMA
  CUtensorMap tm;
  const uint64_t row_elems = static_cast<uint64_t>(3 * heads * head_dim);
  {
    const uint64_t gdim[3] = {row_elems, static_cast<uint64_t>(seq_len), static_cast<uint64_t>(batch)};
    const uint64_t gstr[2] = {row_elems * 2, row_elems * 2 * static_cast<uint64_t>(seq_len)};
    const uint32_t box[3] = {64, 128, 1};
    const uint32_t estr[3] = {1, 1, 1};
    const int before = mgpuGetLastError();
    mgpuTensorMapEncodeTiled(&tm, dtype == MGPU_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                             3, const_cast<void *>(qkv), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (before == 0 && mgpuGetLastError() != 0) return;
  }
  // the output as (column, position, sequence) in boxes of 64 columns x 32 rows: a warp's
  // rows past the end of the sequence are clipped instead of landing in the next sequence
  CUtensorMap tmo;
  {
    const uint64_t out_row = static_cast<uint64_t>(heads * head_dim);
    const uint64_t gdim[3] = {out_row, static_cast<uint64_t>(seq_len), static_cast<uint64_t>(batch)};
    const uint64_t gstr[2] = {out_row * 2, out_row * 2 * static_cast<uint64_t>(seq_len)};
    const uint32_t box[3] = {64, 32, 1};
    const uint32_t estr[3] = {1, 1, 1};
    const int before = mgpuGetLastError();
    mgpuTensorMapEncodeTiled(&tmo, dtype == MGPU_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                             3, out, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (before == 0 && mgpuGetLastError() != 0) return;
  }
  AttnParams p;
  p.seq_lens = seq_lens;
  p.out = out;
  p.batch = static_cast<int>(batch);
  p.seq = static_cast<int>(seq_len);
  p.heads = static_cast<int>(heads);
  p.causal = causal ? 1 : 0;
  p.scale_log2e = 1.4426950408889634f / sqrtf(static_cast<float>(head_dim));
  p.err = err;
  const int64_t n_items = q_tiles * heads * batch;
  if (n_items > 0x7fffffff) { fail("mgpuAttention: shape too large"); return; }
  cudaStream_t s = as_stream(stream);
  ProfileScope prof(kCatAttention, s);
  // MDC_ATTN_GENERAL=1 runs the general kernel at head_dim 64 too (for measurements)
  static const bool general64 = getenv("MDC_ATTN_GENERAL") && atoi(getenv("MDC_ATTN_GENERAL")) != 0;
  if (dtype == MGPU_DTYPE_F16) {
    if (head_dim == 128) launch_attention<__half, 128>(tm, tmo, p, n_items, di, s);
    else if (general64) launch_attention<__half, 64>(tm, tmo, p, n_items, di, s);
    else launch_attention64<__half>(tm, tmo, p, n_items, di, s);
  } else {
    if (head_dim == 128) launch_attention<__nv_bfloat16, 128>(tm, tmo, p, n_items, di, s);
    else if (general64) launch_attention<__nv_bfloat16, 64>(tm, tmo, p, n_items, di, s);
    else launch_attention64<__nv_bfloat16>(tm, tmo, p, n_items, di, s);
  }
  launched("attention_tcgen05_kernel");
}
