// Lowered graph of a post-LN transformer encoder stack (hidden 768, 12 heads x 64, FFN
// 3072, exact GELU, fp16 inside): out[B,S,768] = Stack(x[B,S,768], lens[B]).
//
// A compiled model carries its weights as constants inside the model library; here they
// are generated on first use from a fixed seed (i.i.d. N(0, 0.02), biases 0, LayerNorm
// gamma 1 / beta 0), uploaded and packed once, and kept for later calls - the role of a
// constant-weight cache.  mdc_graph_fill_normal exposes the generator so a checker can
// rebuild the very same weights.  Environment: MDC_GRAPH_LAYERS (default 1) selects the
// depth.  lens holds the valid length of every sequence as fp32 (the runner only passes
// fp32 tensors, lib/Runtime/RuntimeUtil.cpp:9-23); a value <= 0 or >= S means full length.
#include <cmath>
#include <vector>

#include "graph_common.h"

namespace {
constexpr int64_t kD = 768, kF = 3072, kH = 12;

inline uint64_t splitmix64(uint64_t &s) {
  uint64_t z = (s += 0x9e3779b97f4a7c15ull);
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

void *g_stack = nullptr;
int64_t g_layers = 0;
}  // namespace

// dst[i] = std * z_i with z_i standard normal (Box-Muller over a splitmix64 stream)
MDC_GRAPH_EXPORT void mdc_graph_fill_normal(float *dst, int64_t n, uint64_t seed, float stddev) {
  uint64_t s = seed * 0x2545f4914f6cdd1dull + 0x1234567ull;
  for (int64_t i = 0; i < n; i += 2) {
    const double u1 = (static_cast<double>(splitmix64(s) >> 11) + 1.0) / 9007199254740993.0;
    const double u2 = static_cast<double>(splitmix64(s) >> 11) / 9007199254740992.0;
    const double r = std::sqrt(-2.0 * std::log(u1));
    dst[i] = static_cast<float>(stddev * r * std::cos(6.283185307179586 * u2));
    if (i + 1 < n) dst[i + 1] = static_cast<float>(stddev * r * std::sin(6.283185307179586 * u2));
  }
}

// seed of weight matrix `which` (0 qkv, 1 proj, 2 ffn1, 3 ffn2) of layer l
MDC_GRAPH_EXPORT uint64_t mdc_graph_weight_seed(int64_t layer, int64_t which) {
  return 1000ull + static_cast<uint64_t>(layer) * 4ull + static_cast<uint64_t>(which);
}

MDC_GRAPH_EXPORT int64_t mdc_graph_num_layers(void) {
  const char *e = getenv("MDC_GRAPH_LAYERS");
  const long v = e ? atol(e) : 1;
  return v > 0 ? v : 1;
}

static void build_stack(mgpu_stream_t s) {
  g_layers = mdc_graph_num_layers();
  g_stack = mgpuEncoderStackCreate(g_layers, kD, kF, kH, false, false, MGPU_ACT_GELU_ERF, MGPU_DTYPE_F16, 1e-5f);
  if (!g_stack) return;
  const int64_t shapes[4][2] = {{kD, 3 * kD}, {kD, kD}, {kD, kF}, {kF, kD}};
  std::vector<float> host(static_cast<size_t>(kD) * kF);
  for (int64_t l = 0; l < g_layers; ++l) {
    float *dev[4];
    for (int w = 0; w < 4; ++w) {
      const int64_t n = shapes[w][0] * shapes[w][1];
      mdc_graph_fill_normal(host.data(), n, mdc_graph_weight_seed(l, w), 0.02f);
      dev[w] = upload(host.data(), n, s);
      mgpuStreamSynchronize(s);  // host staging buffer is reused
    }
    mgpuEncoderStackSetLayer(g_stack, l, dev[0], nullptr, dev[1], nullptr, dev[2], nullptr, dev[3], nullptr,
                             nullptr, nullptr, nullptr, nullptr, s);
    for (int w = 0; w < 4; ++w) mgpuMemFree(dev[w], s);
  }
  mgpuStreamSynchronize(s);
}

MDC_GRAPH_EXPORT void _mlir_ciface_main_graph(MemRef<3> *out, MemRef<3> *x, MemRef<1> *lens) {
  const int64_t B = x->sizes[0], S = x->sizes[1], d = x->sizes[2];
  float *host_out = alloc_result<3>(out, x->sizes);
  if (d != kD) {
    mgpuSetLastError(-1, "encoder graph: hidden size must be 768");
    return;
  }
  GraphStreams st;
  if (!g_stack) build_stack(st.data);
  if (!g_stack) { st.end(); return; }
  float *dx = upload(x->data(), B * S * d, st.data);
  std::vector<int32_t> li(static_cast<size_t>(B));
  bool ragged = false;
  for (int64_t b = 0; b < B; ++b) {
    const float v = lens ? lens->data()[b] : 0.f;
    li[b] = (v <= 0.f || v >= static_cast<float>(S)) ? static_cast<int32_t>(S) : static_cast<int32_t>(v);
    ragged |= li[b] != S;
  }
  int32_t *dl = nullptr;
  if (ragged) {
    dl = static_cast<int32_t *>(mgpuMemAlloc(static_cast<uint64_t>(B) * 4, st.data));
    mgpuMemcpy(dl, li.data(), static_cast<size_t>(B) * 4, st.data);
  }
  float *dy = static_cast<float *>(mgpuMemAlloc(static_cast<uint64_t>(B) * S * d * 4, st.data));
  st.data_to_kernel();
  mgpuEncoderStackRun(g_stack, dx, dl, dy, B, S, st.kernel);
  st.kernel_to_data();
  mgpuMemcpy(host_out, dy, static_cast<size_t>(B) * S * d * 4, st.data);
  mgpuMemFree(dx, st.data);
  if (dl) mgpuMemFree(dl, st.data);
  mgpuMemFree(dy, st.data);
  st.end();
}
