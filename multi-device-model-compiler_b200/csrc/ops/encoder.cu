// Transformer encoder layer / stack orchestration on top of the hand-written kernels.
//
// Replaces mgpuLLMDecodingContextLayer (lib/Kernels/GPU/LLM.cu:26-158).  The reference
// re-casts every weight fp32->fp16 on every call, allocates about twenty temporaries per
// call and runs cast / LayerNorm / 4 cuBLASLt Gemms / a vendored fused-MHA cubin on two
// streams.  Here the weights are packed once into the tensor-core operand layout and kept
// in a handle; a layer is 7 kernel launches on one stream:
//   post-LN: qkv = Gemm(x) ; att = Attention(qkv) ; a = Gemm(att)+bias+x ; y1 = LN1(a) ;
//            f1 = act(Gemm(y1)+b1) ; f2 = Gemm(f1)+b2+y1 ; y = LN2(f2)
//   pre-LN : n1 = LN1(x) ; qkv = Gemm(n1) ; att ; a = Gemm(att)+bias+x ; n2 = LN2(a) ;
//            f1 = act(Gemm(n2)+b1) ; y = Gemm(f1)+b2+a
// Bias, activation, residual add and the output type conversion ride in the Gemm epilogue;
// attention reads the packed QKV rows directly (no split / transpose kernel, the job of
// lib/Kernels/GPU/Transpose.cu:6-85).  Activations between kernels are 16-bit, statistics
// and accumulation fp32; the boundary is fp32 like the reference's.
#include <cstdlib>
#include <vector>

#include "ops_common.h"

namespace mdc {

struct LayerWeights {
  void *wqkv = nullptr, *wo = nullptr, *w1 = nullptr, *w2 = nullptr;  // 16-bit [N, K]
  float *bqkv = nullptr, *bo = nullptr, *b1 = nullptr, *b2 = nullptr;
  float *ln1_g = nullptr, *ln1_b = nullptr, *ln2_g = nullptr, *ln2_b = nullptr;
};

struct Workspace {
  int64_t tokens = 0;
  void *cur = nullptr, *qkv = nullptr, *att = nullptr, *a = nullptr, *n1 = nullptr, *f1 = nullptr;
};

struct EncoderStack {
  int64_t layers_n = 0, d = 0, F = 0, H = 0;
  bool norm_first = false, causal = false;
  int32_t act = MGPU_ACT_GELU_ERF, dtype = MGPU_DTYPE_F16;
  float eps = 1e-5f;
  std::vector<LayerWeights> layers;
  Workspace ws;
  // host-buffer pipeline state
  cudaStream_t s_in = nullptr, s_comp = nullptr, s_out = nullptr;
  cudaEvent_t ev_in[2] = {nullptr, nullptr}, ev_comp[2] = {nullptr, nullptr}, ev_out[2] = {nullptr, nullptr};
  void *x_dev[2] = {nullptr, nullptr}, *y_dev[2] = {nullptr, nullptr};
  int32_t *lens_dev[2] = {nullptr, nullptr};
  int64_t pipe_tokens = 0, pipe_seqs = 0;  // capacity of the IO buffers (tokens) and of the lengths buffers
  bool slot_used[2] = {false, false};  // the slot's events have been recorded at least once
  int64_t tickets = 0;                 // submissions made through mgpuEncoderStackSubmitHost
  // recorded at the end of every run; the next run (on any stream) waits for it, because
  // all runs of a stack share one activation workspace
  cudaEvent_t done_ev = nullptr;
  bool used = false;
  // CUDA graphs of whole runs, keyed by the run's pointers and shape (see run_stack_replayed)
  struct RunGraph {
    const float *x = nullptr;
    const int32_t *lens = nullptr;
    float *y = nullptr;
    int64_t B = 0, S = 0;
    int seen = 0;                    // eager runs with this key so far
    cudaGraphExec_t exec = nullptr;  // set once captured
  };
  std::vector<RunGraph> graphs;
  bool graphs_off = false;  // a capture failed: stay eager
};

static void drop_graphs(EncoderStack *st) {
  for (auto &g : st->graphs)
    if (g.exec) cudaGraphExecDestroy(g.exec);
  st->graphs.clear();
}

static void order_after_previous(EncoderStack *st, void *stream) {
  if (!st->done_ev) check_cuda(cudaEventCreateWithFlags(&st->done_ev, cudaEventDisableTiming), "event");
  if (st->used && st->done_ev) cudaStreamWaitEvent(as_stream(stream), st->done_ev, 0);
}
static void mark_run_done(EncoderStack *st, void *stream) {
  if (st->done_ev) cudaEventRecord(st->done_ev, as_stream(stream));
  st->used = true;
}

static void free_ws(Workspace &w, void *stream) {
  // (graphs captured over these buffers are dropped by the callers that own a stack)
  void **p[] = {&w.cur, &w.qkv, &w.att, &w.a, &w.n1, &w.f1};
  for (auto q : p) {
    if (*q) mgpuMemFreeAsync(*q, stream);
    *q = nullptr;
  }
  w.tokens = 0;
}

static bool ensure_ws(EncoderStack *st, int64_t tokens, void *stream) {
  Workspace &w = st->ws;
  if (w.tokens >= tokens) return true;
  drop_graphs(st);  // they hold the old buffers' addresses
  free_ws(w, stream);
  const uint64_t T = static_cast<uint64_t>(tokens), d = st->d, F = st->F;
  w.cur = mgpuMemAllocAsync(T * d * 2, stream);
  w.qkv = mgpuMemAllocAsync(T * 3 * d * 2, stream);
  w.att = mgpuMemAllocAsync(T * d * 2, stream);
  w.a = mgpuMemAllocAsync(T * d * 2, stream);
  w.n1 = mgpuMemAllocAsync(T * d * 2, stream);
  w.f1 = mgpuMemAllocAsync(T * F * 2, stream);
  if (!w.cur || !w.qkv || !w.att || !w.a || !w.n1 || !w.f1) {
    free_ws(w, stream);
    fail("encoder stack: out of device memory for the activation workspace");
    return false;
  }
  w.tokens = tokens;
  return true;
}

static float *dup_f32(const float *src, int64_t n, void *stream) {
  if (!src) return nullptr;
  float *dst = static_cast<float *>(mgpuMemAllocAsync(static_cast<uint64_t>(n) * 4, stream));
  if (dst) check_cuda(cudaMemcpyAsync(dst, src, n * 4, cudaMemcpyDeviceToDevice, as_stream(stream)), "copy bias");
  return dst;
}

static void *pack(const float *w, int64_t K, int64_t N, int32_t dtype, void *stream) {
  if (!w) return nullptr;
  void *dst = mgpuMemAllocAsync(static_cast<uint64_t>(N) * K * 2, stream);
  if (dst) mgpuPackWeight(w, dst, K, N, dtype, stream);
  return dst;
}

static void free_layer(LayerWeights &lw, void *stream) {
  void *p[] = {lw.wqkv, lw.wo, lw.w1, lw.w2, lw.bqkv, lw.bo, lw.b1, lw.b2, lw.ln1_g, lw.ln1_b, lw.ln2_g, lw.ln2_b};
  for (void *q : p)
    if (q) mgpuMemFreeAsync(q, stream);
  lw = LayerWeights();
}

static void destroy_stack(EncoderStack *st, void *stream) {
  if (!st) return;
  drop_graphs(st);
  for (auto &lw : st->layers) free_layer(lw, stream);
  free_ws(st->ws, stream);
  for (int i = 0; i < 2; ++i) {
    if (st->x_dev[i]) mgpuMemFreeAsync(st->x_dev[i], stream);
    if (st->y_dev[i]) mgpuMemFreeAsync(st->y_dev[i], stream);
    if (st->lens_dev[i]) mgpuMemFreeAsync(st->lens_dev[i], stream);
    if (st->ev_in[i]) cudaEventDestroy(st->ev_in[i]);
    if (st->ev_comp[i]) cudaEventDestroy(st->ev_comp[i]);
    if (st->ev_out[i]) cudaEventDestroy(st->ev_out[i]);
  }
  if (st->done_ev) cudaEventDestroy(st->done_ev);
  if (st->s_in) cudaStreamDestroy(st->s_in);
  if (st->s_comp) cudaStreamDestroy(st->s_comp);
  if (st->s_out) cudaStreamDestroy(st->s_out);
  delete st;
}

// x_f32 != nullptr: input is fp32 and is cast first; else `cur` already holds 16-bit input.
// y_f32 receives the fp32 result.
static void run_stack(EncoderStack *st, const float *x_f32, const int32_t *seq_lens, float *y_f32,
                      int64_t B, int64_t S, void *stream) {
  const int64_t T = B * S, d = st->d, F = st->F;
  const int32_t dt = st->dtype;
  Workspace &w = st->ws;
  mgpuCast(x_f32, MGPU_DTYPE_F32, w.cur, dt, T * d, stream);
  const int64_t L = st->layers_n;
  for (int64_t l = 0; l < L; ++l) {
    const LayerWeights &lw = st->layers[l];
    const bool last = (l + 1 == L);
    if (!lw.wqkv || !lw.wo || !lw.w1 || !lw.w2) {
      fail("encoder stack: layer weights were not set");
      return;
    }
    if (st->norm_first) {
      mgpuLayerNormEx(w.cur, nullptr, lw.ln1_g, lw.ln1_b, nullptr, w.n1, st->eps, T, d, dt, dt, stream);
      mgpuMatmulEx16(w.n1, lw.wqkv, lw.bqkv, nullptr, w.qkv, T, 3 * d, d, dt, dt, MGPU_ACT_NONE, stream);
      mgpuAttention(w.qkv, seq_lens, w.att, B, S, st->H, d / st->H, st->causal, dt, stream);
      mgpuMatmulEx16(w.att, lw.wo, lw.bo, w.cur, w.a, T, d, d, dt, dt, MGPU_ACT_NONE, stream);
      mgpuLayerNormEx(w.a, nullptr, lw.ln2_g, lw.ln2_b, nullptr, w.n1, st->eps, T, d, dt, dt, stream);
      mgpuMatmulEx16(w.n1, lw.w1, lw.b1, nullptr, w.f1, T, F, d, dt, dt, st->act, stream);
      if (last)
        mgpuMatmulEx16(w.f1, lw.w2, lw.b2, w.a, y_f32, T, d, F, dt, MGPU_DTYPE_F32, MGPU_ACT_NONE, stream);
      else
        mgpuMatmulEx16(w.f1, lw.w2, lw.b2, w.a, w.cur, T, d, F, dt, dt, MGPU_ACT_NONE, stream);
    } else {
      mgpuMatmulEx16(w.cur, lw.wqkv, lw.bqkv, nullptr, w.qkv, T, 3 * d, d, dt, dt, MGPU_ACT_NONE, stream);
      mgpuAttention(w.qkv, seq_lens, w.att, B, S, st->H, d / st->H, st->causal, dt, stream);
      mgpuMatmulEx16(w.att, lw.wo, lw.bo, w.cur, w.a, T, d, d, dt, dt, MGPU_ACT_NONE, stream);
      mgpuLayerNormEx(w.a, nullptr, lw.ln1_g, lw.ln1_b, nullptr, w.n1, st->eps, T, d, dt, dt, stream);
      mgpuMatmulEx16(w.n1, lw.w1, lw.b1, nullptr, w.f1, T, F, d, dt, dt, st->act, stream);
      mgpuMatmulEx16(w.f1, lw.w2, lw.b2, w.n1, w.a, T, d, F, dt, dt, MGPU_ACT_NONE, stream);
      if (last)
        mgpuLayerNormEx(w.a, nullptr, lw.ln2_g, lw.ln2_b, nullptr, y_f32, st->eps, T, d, dt, MGPU_DTYPE_F32, stream);
      else
        mgpuLayerNormEx(w.a, nullptr, lw.ln2_g, lw.ln2_b, nullptr, w.cur, st->eps, T, d, dt, dt, stream);
    }
  }
}

// A run whose pointers and shape have been seen before is replayed as a CUDA graph: the 85
// launches of a 12-layer step (with their tensor-map encodes and launch attributes) cost the
// host 0.5 - 2.7 ms per step, a graph launch a few microseconds, and the device gets the whole
// chain, programmatic dependencies included, in one piece.  The first run with a key is eager
// (it also does the one-time set-up that cannot be captured: function attributes, symbol
// look-ups), the second is captured, later ones replay.  Not while profiling (per-kernel
// events), not inside a caller's own capture; MDC_GRAPHS=0 turns it off.
static bool graphs_enabled() {
  static const bool on = !(getenv("MDC_GRAPHS") && atoi(getenv("MDC_GRAPHS")) == 0);
  return on;
}
static void run_stack_replayed(EncoderStack *st, const float *x, const int32_t *lens, float *y, int64_t B, int64_t S,
                               void *stream) {
  cudaStream_t s = as_stream(stream);
  bool eligible = graphs_enabled() && !st->graphs_off && !g_profiling && s != nullptr;
  if (eligible) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
      (void)cudaGetLastError();
      eligible = false;
    }
  }
  if (!eligible) {
    run_stack(st, x, lens, y, B, S, stream);
    return;
  }
  EncoderStack::RunGraph *g = nullptr;
  for (auto &c : st->graphs)
    if (c.x == x && c.lens == lens && c.y == y && c.B == B && c.S == S) g = &c;
  if (!g) {
    if (st->graphs.size() >= 8) {  // a caller that keeps changing buffers: forget the oldest
      if (st->graphs.front().exec) cudaGraphExecDestroy(st->graphs.front().exec);
      st->graphs.erase(st->graphs.begin());
    }
    EncoderStack::RunGraph fresh;
    fresh.x = x, fresh.lens = lens, fresh.y = y, fresh.B = B, fresh.S = S;
    st->graphs.push_back(fresh);
    g = &st->graphs.back();
  }
  if (g->exec) {
    if (check_cuda(cudaGraphLaunch(g->exec, s), "cudaGraphLaunch")) {
      g_launch_count.fetch_add(static_cast<uint64_t>(st->layers_n) * 7 + 1, std::memory_order_relaxed);
      return;
    }
    st->graphs_off = true;
    run_stack(st, x, lens, y, B, S, stream);
    return;
  }
  if (g->seen++ == 0 || mgpuGetLastError() != 0) {
    run_stack(st, x, lens, y, B, S, stream);
    return;
  }
  // second run with this key: capture it, then launch what was captured
  cudaGraph_t graph = nullptr;
  if (cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
    (void)cudaGetLastError();
    st->graphs_off = true;
    run_stack(st, x, lens, y, B, S, stream);
    return;
  }
  const uint64_t launches_before = g_launch_count.load(std::memory_order_relaxed);
  run_stack(st, x, lens, y, B, S, stream);
  const cudaError_t end = cudaStreamEndCapture(s, &graph);
  g_launch_count.store(launches_before, std::memory_order_relaxed);  // captured, not yet launched
  cudaGraphExec_t exec = nullptr;
  if (end != cudaSuccess || !graph || mgpuGetLastError() != 0 ||
      cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) {
    (void)cudaGetLastError();
    if (graph) cudaGraphDestroy(graph);
    st->graphs_off = true;
    if (mgpuGetLastError() == 0) run_stack(st, x, lens, y, B, S, stream);
    return;
  }
  cudaGraphDestroy(graph);
  g->exec = exec;
  if (check_cuda(cudaGraphLaunch(exec, s), "cudaGraphLaunch"))
    g_launch_count.fetch_add(static_cast<uint64_t>(st->layers_n) * 7 + 1, std::memory_order_relaxed);
}

static bool valid_config(int64_t L, int64_t d, int64_t F, int64_t H, int32_t act, int32_t dtype) {
  if (L <= 0 || d <= 0 || F <= 0 || H <= 0) { fail("encoder: sizes must be positive"); return false; }
  if (d % H != 0 || (d / H != 64 && d / H != 128)) { fail("encoder: d_model / head_num must be 64 or 128"); return false; }
  if (d % 8 || F % 8) { fail("encoder: d_model and feed_forward_dim must be multiples of 8"); return false; }
  if (!dtype_is16(dtype)) { fail("encoder: dtype must be F16 or BF16"); return false; }
  if (act < MGPU_ACT_NONE || act > MGPU_ACT_GELU_TANH) { fail("encoder: unknown activation"); return false; }
  return true;
}

}  // namespace mdc

using namespace mdc;

MDC_API void *mgpuEncoderStackCreate(int64_t num_layers, int64_t d_model, int64_t feed_forward_dim,
                                     int64_t head_num, bool norm_first, bool causal, int32_t act,
                                     int32_t dtype, float eps) {
  if (!device_info().ok) return nullptr;
  if (!valid_config(num_layers, d_model, feed_forward_dim, head_num, act, dtype)) return nullptr;
  EncoderStack *st = new EncoderStack();
  st->layers_n = num_layers;
  st->d = d_model;
  st->F = feed_forward_dim;
  st->H = head_num;
  st->norm_first = norm_first;
  st->causal = causal;
  st->act = act;
  st->dtype = dtype;
  st->eps = eps;
  st->layers.resize(static_cast<size_t>(num_layers));
  return st;
}

MDC_API void mgpuEncoderStackSetLayer(void *stack, int64_t layer, const float *qkv_weight,
                                      const float *qkv_bias, const float *proj_weight,
                                      const float *proj_bias, const float *ffn1_weight,
                                      const float *ffn1_bias, const float *ffn2_weight,
                                      const float *ffn2_bias, const float *ln1_gamma,
                                      const float *ln1_beta, const float *ln2_gamma,
                                      const float *ln2_beta, void *stream) {
  EncoderStack *st = static_cast<EncoderStack *>(stack);
  if (!st || layer < 0 || layer >= st->layers_n) { fail("mgpuEncoderStackSetLayer: bad handle or layer index"); return; }
  if (!qkv_weight || !proj_weight || !ffn1_weight || !ffn2_weight) { fail("mgpuEncoderStackSetLayer: weight matrices are required"); return; }
  LayerWeights &lw = st->layers[static_cast<size_t>(layer)];
  drop_graphs(st);  // captured runs hold the old weights' addresses
  free_layer(lw, stream);
  const int64_t d = st->d, F = st->F;
  lw.wqkv = pack(qkv_weight, d, 3 * d, st->dtype, stream);
  lw.wo = pack(proj_weight, d, d, st->dtype, stream);
  lw.w1 = pack(ffn1_weight, d, F, st->dtype, stream);
  lw.w2 = pack(ffn2_weight, F, d, st->dtype, stream);
  lw.bqkv = dup_f32(qkv_bias, 3 * d, stream);
  lw.bo = dup_f32(proj_bias, d, stream);
  lw.b1 = dup_f32(ffn1_bias, F, stream);
  lw.b2 = dup_f32(ffn2_bias, d, stream);
  lw.ln1_g = dup_f32(ln1_gamma, d, stream);
  lw.ln1_b = dup_f32(ln1_beta, d, stream);
  lw.ln2_g = dup_f32(ln2_gamma, d, stream);
  lw.ln2_b = dup_f32(ln2_beta, d, stream);
}

MDC_API void mgpuEncoderStackRun(void *stack, const float *x, const int32_t *seq_lens, float *y,
                                 int64_t batch, int64_t seq_len, void *stream) {
  EncoderStack *st = static_cast<EncoderStack *>(stack);
  if (!st) { fail("mgpuEncoderStackRun: null handle"); return; }
  if (batch <= 0 || seq_len <= 0) return;
  order_after_previous(st, stream);
  if (!ensure_ws(st, batch * seq_len, stream)) return;
  run_stack_replayed(st, x, seq_lens, y, batch, seq_len, stream);
  mark_run_done(st, stream);
}

MDC_API void mgpuEncoderStackDestroy(void *stack) {
  EncoderStack *st = static_cast<EncoderStack *>(stack);
  if (!st) return;
  // blocks go back to the pool ordered after everything already queued on the device
  cudaDeviceSynchronize();
  destroy_stack(st, nullptr);
}

// Streams, events and the two sets of device IO buffers of the host-buffer pipeline, sized
// for `per` sequences.  Growing the buffers first drains whatever is still in flight.
static bool ensure_pipe(EncoderStack *st, int64_t per, int64_t seq_len) {
  const int64_t d = st->d;
  if (!st->s_in) {
    bool ok = check_cuda(cudaStreamCreateWithFlags(&st->s_in, cudaStreamNonBlocking), "stream") &&
              check_cuda(cudaStreamCreateWithFlags(&st->s_comp, cudaStreamNonBlocking), "stream") &&
              check_cuda(cudaStreamCreateWithFlags(&st->s_out, cudaStreamNonBlocking), "stream");
    for (int i = 0; ok && i < 2; ++i)
      ok = check_cuda(cudaEventCreateWithFlags(&st->ev_in[i], cudaEventDisableTiming), "event") &&
           check_cuda(cudaEventCreateWithFlags(&st->ev_comp[i], cudaEventDisableTiming), "event") &&
           check_cuda(cudaEventCreateWithFlags(&st->ev_out[i], cudaEventDisableTiming), "event");
    if (!ok) return false;
  }
  if (st->pipe_tokens < per * seq_len || st->pipe_seqs < per) {
    cudaStreamSynchronize(st->s_in);
    cudaStreamSynchronize(st->s_comp);
    cudaStreamSynchronize(st->s_out);
    const int64_t tokens = st->pipe_tokens > per * seq_len ? st->pipe_tokens : per * seq_len;
    const int64_t seqs = st->pipe_seqs > per ? st->pipe_seqs : per;
    drop_graphs(st);
    for (int i = 0; i < 2; ++i) {
      if (st->x_dev[i]) mgpuMemFreeAsync(st->x_dev[i], st->s_comp);
      if (st->y_dev[i]) mgpuMemFreeAsync(st->y_dev[i], st->s_comp);
      if (st->lens_dev[i]) mgpuMemFreeAsync(st->lens_dev[i], st->s_comp);
      const uint64_t bytes = static_cast<uint64_t>(tokens) * d * 4;
      st->x_dev[i] = mgpuMemAllocAsync(bytes, st->s_comp);
      st->y_dev[i] = mgpuMemAllocAsync(bytes, st->s_comp);
      st->lens_dev[i] = static_cast<int32_t *>(mgpuMemAllocAsync(static_cast<uint64_t>(seqs) * 4, st->s_comp));
      if (!st->x_dev[i] || !st->y_dev[i] || !st->lens_dev[i]) {
        st->pipe_tokens = st->pipe_seqs = 0;
        fail("encoder stack: out of device memory for the IO buffers");
        return false;
      }
    }
    st->pipe_tokens = tokens;
    st->pipe_seqs = seqs;
    check_cuda(cudaStreamSynchronize(st->s_comp), "sync");
  }
  order_after_previous(st, st->s_comp);
  return ensure_ws(st, per * seq_len, st->s_comp);
}

// upload -> stack -> download of nb sequences through IO buffer set `set`, each stage on its
// own stream, ordered against the previous user of the same set by events
static void enqueue_host_chunk(EncoderStack *st, int set, const float *x_host, const int32_t *lens_host,
                               float *y_host, int64_t nb, int64_t seq_len) {
  const size_t elems = static_cast<size_t>(nb) * seq_len * st->d;
  if (st->slot_used[set]) cudaStreamWaitEvent(st->s_in, st->ev_comp[set], 0);  // x_dev[set] consumed
  check_cuda(cudaMemcpyAsync(st->x_dev[set], x_host, elems * 4, cudaMemcpyHostToDevice, st->s_in), "H2D");
  if (lens_host)
    check_cuda(cudaMemcpyAsync(st->lens_dev[set], lens_host, nb * 4, cudaMemcpyHostToDevice, st->s_in), "H2D lens");
  cudaEventRecord(st->ev_in[set], st->s_in);
  cudaStreamWaitEvent(st->s_comp, st->ev_in[set], 0);
  if (st->slot_used[set]) cudaStreamWaitEvent(st->s_comp, st->ev_out[set], 0);  // y_dev[set] drained
  run_stack_replayed(st, static_cast<const float *>(st->x_dev[set]), lens_host ? st->lens_dev[set] : nullptr,
                     static_cast<float *>(st->y_dev[set]), nb, seq_len, st->s_comp);
  cudaEventRecord(st->ev_comp[set], st->s_comp);
  mark_run_done(st, st->s_comp);
  cudaStreamWaitEvent(st->s_out, st->ev_comp[set], 0);
  check_cuda(cudaMemcpyAsync(y_host, st->y_dev[set], elems * 4, cudaMemcpyDeviceToHost, st->s_out), "D2H");
  cudaEventRecord(st->ev_out[set], st->s_out);
  st->slot_used[set] = true;
}

MDC_API void mgpuEncoderStackRunHost(void *stack, const float *x_host, const int32_t *seq_lens_host,
                                     float *y_host, int64_t batch, int64_t seq_len, int32_t chunks) {
  EncoderStack *st = static_cast<EncoderStack *>(stack);
  if (!st) { fail("mgpuEncoderStackRunHost: null handle"); return; }
  if (batch <= 0 || seq_len <= 0) return;
  // Chunk sizes.  Only the first chunk's upload and the last chunk's download are exposed
  // (everything else overlaps compute), while small chunks run the kernels less efficiently:
  // so the first and the last chunk are small (batch / 8) and the rest is split evenly.
  if (chunks < 1) chunks = 1;
  if (chunks > batch) chunks = static_cast<int32_t>(batch);
  std::vector<int64_t> sizes;
  if (chunks <= 2 || batch < 16) {
    const int64_t even = (batch + chunks - 1) / chunks;
    for (int64_t b0 = 0; b0 < batch; b0 += even) sizes.push_back(batch - b0 < even ? batch - b0 : even);
  } else {
    const int64_t edge = batch / 8 > 0 ? batch / 8 : 1;
    const int64_t mid = batch - 2 * edge, parts = chunks - 2;
    sizes.push_back(edge);
    for (int64_t i = 0; i < parts; ++i) sizes.push_back(mid / parts + (i < mid % parts ? 1 : 0));
    sizes.push_back(edge);
  }
  int64_t per = 0;  // largest chunk: sizes the device buffers and the workspace
  for (int64_t v : sizes) per = v > per ? v : per;
  if (!ensure_pipe(st, per, seq_len)) return;
  const int64_t d = st->d;
  int n = 0;
  int64_t b0 = 0;
  for (size_t ci = 0; ci < sizes.size(); b0 += sizes[ci], ++ci, ++n) {
    const int64_t nb = sizes[ci];
    if (nb <= 0) continue;
    const size_t off = static_cast<size_t>(b0) * seq_len * d;
    enqueue_host_chunk(st, n & 1, x_host + off, seq_lens_host ? seq_lens_host + b0 : nullptr, y_host + off, nb, seq_len);
  }
  check_cuda(cudaStreamSynchronize(st->s_out), "sync");
  check_cuda(cudaStreamSynchronize(st->s_comp), "sync");
  check_cuda(cudaStreamSynchronize(st->s_in), "sync");
}

// Pipelined form of RunHost for a stream of batches: Submit queues upload, stack and download
// of one whole batch and returns at once; consecutive submissions alternate between the two
// IO buffer sets, so batch i+1 is uploaded while batch i computes and batch i-1 downloads.
MDC_API int64_t mgpuEncoderStackSubmitHost(void *stack, const float *x_host, const int32_t *seq_lens_host,
                                           float *y_host, int64_t batch, int64_t seq_len) {
  EncoderStack *st = static_cast<EncoderStack *>(stack);
  if (!st) { fail("mgpuEncoderStackSubmitHost: null handle"); return -1; }
  if (batch <= 0 || seq_len <= 0 || !x_host || !y_host) { fail("mgpuEncoderStackSubmitHost: empty batch or null buffer"); return -1; }
  if (!ensure_pipe(st, batch, seq_len)) return -1;
  enqueue_host_chunk(st, static_cast<int>(st->tickets & 1), x_host, seq_lens_host, y_host, batch, seq_len);
  return st->tickets++;
}

MDC_API void mgpuEncoderStackWaitHost(void *stack, int64_t ticket) {
  EncoderStack *st = static_cast<EncoderStack *>(stack);
  if (!st) { fail("mgpuEncoderStackWaitHost: null handle"); return; }
  if (ticket < 0 || ticket >= st->tickets) { fail("mgpuEncoderStackWaitHost: unknown ticket"); return; }
  // downloads complete in submission order on one stream: the latest event recorded on the
  // ticket's buffer set is at or after the ticket's own
  check_cuda(cudaEventSynchronize(st->ev_out[ticket & 1]), "wait for the download");
}

MDC_API void mgpuTransformerEncoderLayer(const float *input, const float *qkv_weight, const float *qkv_bias,
                                         const float *proj_weight, const float *proj_bias,
                                         const float *ffn1_weight, const float *ffn1_bias,
                                         const float *ffn2_weight, const float *ffn2_bias,
                                         const float *ln1_gamma, const float *ln1_beta,
                                         const float *ln2_gamma, const float *ln2_beta,
                                         const int32_t *seq_lens, float *output, int64_t batch,
                                         int64_t seq_len, int64_t d_model, int64_t feed_forward_dim,
                                         int64_t head_num, bool norm_first, bool causal, int32_t act,
                                         int32_t dtype, float eps, void *stream) {
  if (batch <= 0 || seq_len <= 0) return;
  if (!device_info().ok) return;
  if (!valid_config(1, d_model, feed_forward_dim, head_num, act, dtype)) return;
  if (!qkv_weight || !proj_weight || !ffn1_weight || !ffn2_weight) { fail("mgpuTransformerEncoderLayer: weight matrices are required"); return; }
  // A one-call stack that owns nothing but its workspace: biases and LayerNorm parameters are
  // read where the caller has them, and a weight that is a copy of a registered constant
  // comes packed from the constant cache (the reference re-casts all four weights on every
  // call, LLM.cu:56-57,86-90,102-106,126-130); other weights are packed into pool blocks that
  // go back in stream order, as the reference does with its temporaries (LLM.cu:143-154).
  EncoderStack st;
  st.layers_n = 1;
  st.d = d_model;
  st.F = feed_forward_dim;
  st.H = head_num;
  st.norm_first = norm_first;
  st.causal = causal;
  st.act = act;
  st.dtype = dtype;
  st.eps = eps;
  st.layers.resize(1);
  LayerWeights &lw = st.layers[0];
  const int64_t d = d_model, F = feed_forward_dim;
  bool cached[4] = {false, false, false, false};
  lw.wqkv = packed_weight(qkv_weight, d, 3 * d, dtype, stream, &cached[0]);
  lw.wo = packed_weight(proj_weight, d, d, dtype, stream, &cached[1]);
  lw.w1 = packed_weight(ffn1_weight, d, F, dtype, stream, &cached[2]);
  lw.w2 = packed_weight(ffn2_weight, F, d, dtype, stream, &cached[3]);
  lw.bqkv = const_cast<float *>(qkv_bias);
  lw.bo = const_cast<float *>(proj_bias);
  lw.b1 = const_cast<float *>(ffn1_bias);
  lw.b2 = const_cast<float *>(ffn2_bias);
  lw.ln1_g = const_cast<float *>(ln1_gamma);
  lw.ln1_b = const_cast<float *>(ln1_beta);
  lw.ln2_g = const_cast<float *>(ln2_gamma);
  lw.ln2_b = const_cast<float *>(ln2_beta);
  if (lw.wqkv && lw.wo && lw.w1 && lw.w2) {
    if (ensure_ws(&st, batch * seq_len, stream)) run_stack(&st, input, seq_lens, output, batch, seq_len, stream);
  } else {
    fail("mgpuTransformerEncoderLayer: out of device memory for the packed weights");
  }
  void *packed[4] = {lw.wqkv, lw.wo, lw.w1, lw.w2};
  for (int i = 0; i < 4; ++i)
    if (packed[i] && !cached[i]) mgpuMemFreeAsync(packed[i], stream);
  free_ws(st.ws, stream);
}

// Legacy entry point: LayerNorm without affine, no QKV bias, full-length sequences, fp16.
MDC_API void mgpuLLMDecodingContextLayer(float *input, float *qkv, float *gemm_weight, float *gemm_bias,
                                         float *ffn1_weight, float *ffn1_bias, float *ffn2_weight,
                                         float *ffn2_bias, float *output, int64_t batch, int64_t seq_len,
                                         int64_t d_model, int64_t feed_forward_dim, int64_t head_num,
                                         bool norm_first, bool is_casual, bool is_relu, void *stream) {
  mgpuTransformerEncoderLayer(input, qkv, nullptr, gemm_weight, gemm_bias, ffn1_weight, ffn1_bias,
                              ffn2_weight, ffn2_bias, nullptr, nullptr, nullptr, nullptr, nullptr, output,
                              batch, seq_len, d_model, feed_forward_dim, head_num, norm_first, is_casual,
                              is_relu ? MGPU_ACT_RELU : MGPU_ACT_GELU_ERF, MGPU_DTYPE_F16, 1e-5f, stream);
}
