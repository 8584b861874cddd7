// Lowered graph of ONNX Gemm / MatMul+Add: out[M,N] = in[M,K] . W[K,N] + bias[N], the
// device.matmul call sequence (lib/Conversion/ConvertDeviceToLLVM/ConvertDeviceToLLVM.cpp:
// 410-455: M = product of the leading dims, K = last dim of the input, N = last dim of W).
// The weight arrives already transposed to [K,N] as the compiler leaves it
// (lib/Conversion/ConvertTosaToDevice/Matmul.cpp:57-70).
#include "graph_common.h"

MDC_GRAPH_EXPORT void _mlir_ciface_main_graph(MemRef<2> *out, MemRef<2> *in, MemRef<2> *w, MemRef<1> *bias) {
  const int64_t M = in->sizes[0], K = in->sizes[1], N = w->sizes[1];
  const intptr_t osz[2] = {static_cast<intptr_t>(M), static_cast<intptr_t>(N)};
  float *host_out = alloc_result<2>(out, osz);
  GraphStreams st;
  float *din = upload(in->data(), M * K, st.data);
  float *dw = upload(w->data(), K * N, st.data);
  float *db = upload(bias->data(), N, st.data);
  float *dout = static_cast<float *>(mgpuMemAlloc(static_cast<uint64_t>(M) * N * 4, st.data));
  st.data_to_kernel();
  mgpuMatmul(din, dw, db, dout, M, N, K, st.kernel);
  st.kernel_to_data();
  mgpuMemcpy(host_out, dout, static_cast<size_t>(M) * N * 4, st.data);
  mgpuMemFree(din, st.data);
  mgpuMemFree(dw, st.data);
  mgpuMemFree(db, st.data);
  mgpuMemFree(dout, st.data);
  st.end();
}
