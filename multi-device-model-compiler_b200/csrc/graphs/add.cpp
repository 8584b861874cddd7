// Lowered graph of a single ONNX Add (C = A + B, rank-3 fp32), the graph of
// test/End2End/GPU/add.mlir:4-5 and examples/add.mlir:1-6.  The elementwise kernel is
// fetched by name from the runtime's module interface and launched with a raw launch, the
// way generated kernels are (lib/Dialect/Device/IR/GPUOffloadingAttr.cpp:283-304).
#include "graph_common.h"

MDC_GRAPH_EXPORT void _mlir_ciface_main_graph(MemRef<3> *out, MemRef<3> *a, MemRef<3> *b) {
  int64_t n = a->count();
  float *host_out = alloc_result<3>(out, a->sizes);
  GraphStreams st;
  float *da = upload(a->data(), n, st.data);
  float *db = upload(b->data(), n, st.data);
  float *dc = static_cast<float *>(mgpuMemAlloc(static_cast<uint64_t>(n) * 4, st.data));
  st.data_to_kernel();
  mgpu_function_t fn = mgpuModuleGetFunction("mdc_add_f32");
  intptr_t grid = 1, block = 1;
  mgpuBuiltinLaunchShape(n, &grid, &block);
  void *args[] = {&da, &db, &dc, &n};
  mgpuLaunchKernel(fn, grid, 1, 1, block, 1, 1, 0, st.kernel, args, nullptr);
  st.kernel_to_data();
  mgpuMemcpy(host_out, dc, static_cast<size_t>(n) * 4, st.data);
  mgpuMemFree(da, st.data);
  mgpuMemFree(db, st.data);
  mgpuMemFree(dc, st.data);
  st.end();
}
