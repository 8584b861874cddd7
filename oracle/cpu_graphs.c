/*
 * CPU "lowered graph" modules for the runner tests (TEST INFRASTRUCTURE, not product).
 * Each exports _mlir_ciface_main_graph with the memref calling convention of
 * doc/runtime.md:7-9 and computes on the host with the oracle, which is what a graph
 * compiled by the reference's CPU pipeline does (examples/add.ll:80-104 for Add; mcpuMatmul,
 * lib/Kernels/CPU/Ops.cpp:34-80, for Gemm).  Built three times with -DGRAPH_ADD,
 * -DGRAPH_GEMM, -DGRAPH_LAYERNORM.
 */
#include <stdint.h>
#include <stdlib.h>

void oracle_add_f32(const float *a, const float *b, float *c, int64_t n);
void oracle_matmul(const float *in, const float *w, const float *bias, float *out, int64_t M,
                   int64_t N, int64_t K, int round_mode, int accum64);
void oracle_layernorm(const float *x, const float *gamma, const float *beta, float *y, float eps,
                      int64_t m, int64_t n);

#define MEMREF(N) struct { float *allocated; float *aligned; intptr_t offset; intptr_t sizes[N]; intptr_t strides[N]; }
typedef MEMREF(1) memref1;
typedef MEMREF(2) memref2;
typedef MEMREF(3) memref3;

static float *result(float **allocated, float **aligned, intptr_t *offset, int64_t n) {
  size_t bytes = ((size_t)n * sizeof(float) + 63) / 64 * 64;
  float *p = (float *)aligned_alloc(64, bytes ? bytes : 64);
  *allocated = *aligned = p;
  *offset = 0;
  return p;
}

#if defined(GRAPH_ADD)
void _mlir_ciface_main_graph(memref3 *out, memref3 *a, memref3 *b) {
  int64_t n = 1;
  for (int i = 2; i >= 0; --i) { out->sizes[i] = a->sizes[i]; out->strides[i] = n; n *= a->sizes[i]; }
  float *c = result(&out->allocated, &out->aligned, &out->offset, n);
  oracle_add_f32(a->aligned + a->offset, b->aligned + b->offset, c, n);
}
#elif defined(GRAPH_GEMM)
void _mlir_ciface_main_graph(memref2 *out, memref2 *in, memref2 *w, memref1 *bias) {
  const int64_t M = in->sizes[0], K = in->sizes[1], N = w->sizes[1];
  out->sizes[0] = M; out->sizes[1] = N; out->strides[0] = N; out->strides[1] = 1;
  float *c = result(&out->allocated, &out->aligned, &out->offset, M * N);
  oracle_matmul(in->aligned + in->offset, w->aligned + w->offset, bias->aligned + bias->offset, c, M, N, K, 0, 0);
}
#elif defined(GRAPH_LAYERNORM)
void _mlir_ciface_main_graph(memref3 *out, memref3 *x, memref1 *gamma, memref1 *beta) {
  int64_t n = 1;
  for (int i = 2; i >= 0; --i) { out->sizes[i] = x->sizes[i]; out->strides[i] = n; n *= x->sizes[i]; }
  float *y = result(&out->allocated, &out->aligned, &out->offset, n);
  oracle_layernorm(x->aligned + x->offset, gamma->aligned + gamma->offset, beta->aligned + beta->offset, y,
                   1e-5f, x->sizes[0] * x->sizes[1], x->sizes[2]);
}
#endif
