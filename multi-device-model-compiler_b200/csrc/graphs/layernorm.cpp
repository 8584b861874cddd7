// Lowered graph of a LayerNorm over the last dimension of a rank-3 fp32 tensor with affine
// parameters (eps 1e-5, the value the reference layer uses, lib/Kernels/GPU/LLM.cu:51-52).
#include "graph_common.h"

MDC_GRAPH_EXPORT void _mlir_ciface_main_graph(MemRef<3> *out, MemRef<3> *x, MemRef<1> *gamma, MemRef<1> *beta) {
  const int64_t n = x->sizes[2], m = x->sizes[0] * x->sizes[1];
  float *host_out = alloc_result<3>(out, x->sizes);
  GraphStreams st;
  float *dx = upload(x->data(), m * n, st.data);
  float *dg = upload(gamma->data(), n, st.data);
  float *db = upload(beta->data(), n, st.data);
  float *dy = static_cast<float *>(mgpuMemAlloc(static_cast<uint64_t>(m) * n * 4, st.data));
  st.data_to_kernel();
  mgpuLayerNormF32(dx, dg, db, dy, 1e-5f, m, n, st.kernel);
  st.kernel_to_data();
  mgpuMemcpy(host_out, dy, static_cast<size_t>(m) * n * 4, st.data);
  mgpuMemFree(dx, st.data);
  mgpuMemFree(dg, st.data);
  mgpuMemFree(db, st.data);
  mgpuMemFree(dy, st.data);
  st.end();
}
