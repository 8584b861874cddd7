// multi-device-gpu-runner: loads a lowered model library, calls its graph entry point with
// memref descriptors built from the command line, saves output 0 and times re-runs with
// GPU events.  Same command line as the reference's tool
// (tools/multi-device-gpu-runner/multi-device-gpu-runner.cpp:16-41, lib/Runtime/ModelInfo.cpp:13-28):
//   multi-device-gpu-runner <lib> [--func NAME] [--out-data FILE] [--rerun N] [--ops FILE]
//                           [--input a_b_c,...] [--output a_b_c] [--data f1,f2,...]
// Additions: --gpus N shards dimension 0 (the batch) of input 0 and output 0 over N worker
// processes, one per GPU, every other input replicated; no collective runs inside the
// graph and the only exchange is the final gather of output rows, done by each worker
// writing its slice of the output file.  --json prints one machine-readable result line.
// --constants treats every input after the first as model constants (weights): they are
// registered with the runtime's constant cache, so re-runs upload them once.
// --timeout SECONDS bounds how long the parent waits for a worker before it reports it.
// --device cpu runs a graph that needs no GPU: no CUDA call is made and re-runs are timed
// with the host clock, which is what the reference's multi-device-cpu-runner does
// (tools/multi-device-cpu-runner/multi-device-cpu-runner.cpp:70-82).  The graph library
// decides what is computed; the runner itself never computes anything.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <dlfcn.h>
#include <fcntl.h>
#include <malloc.h>
#include <string>
#include <sys/wait.h>
#include <unistd.h>
#include <vector>

#include "../host/host_runtime.h"
#include "mdc_gpu_ops.h"
#include "mdc_gpu_runtime.h"

void gpuOpsInit();
void gpuOpsDeinit();

using namespace multi_device;

namespace {

struct Options {
  std::string lib, func = "_mlir_ciface_main_graph", out_data, ops = "./ops.cubin";
  std::string input = "3_640_640,3_640_640", output = "3_640_640";
  std::vector<std::string> data;
  int rerun = 0, gpus = 1, timeout_s = 600;
  bool json = false, cpu = false, constants = false;
};

bool take_value(int argc, char **argv, int &i, const char *name, std::string *out) {
  const std::string a = argv[i];
  const std::string flag = std::string("--") + name, flag1 = std::string("-") + name;
  if (a == flag || a == flag1) {
    if (i + 1 >= argc) { fprintf(stderr, "%s needs a value\n", a.c_str()); exit(1); }
    *out = argv[++i];
    return true;
  }
  for (const std::string &f : {flag + "=", flag1 + "="})
    if (a.compare(0, f.size(), f) == 0) { *out = a.substr(f.size()); return true; }
  return false;
}

bool parse(int argc, char **argv, Options *o) {
  for (int i = 1; i < argc; ++i) {
    std::string v;
    if (take_value(argc, argv, i, "func", &o->func)) continue;
    if (take_value(argc, argv, i, "out-data", &o->out_data)) continue;
    if (take_value(argc, argv, i, "ops", &o->ops)) continue;
    if (take_value(argc, argv, i, "input", &o->input)) continue;
    if (take_value(argc, argv, i, "output", &o->output)) continue;
    if (take_value(argc, argv, i, "rerun", &v)) { o->rerun = atoi(v.c_str()); continue; }
    if (take_value(argc, argv, i, "gpus", &v)) { o->gpus = atoi(v.c_str()); continue; }
    if (take_value(argc, argv, i, "timeout", &v)) { o->timeout_s = atoi(v.c_str()); continue; }
    if (take_value(argc, argv, i, "data", &v)) {
      size_t start = 0;
      while (true) {
        const size_t pos = v.find(',', start);
        o->data.push_back(v.substr(start, pos == std::string::npos ? std::string::npos : pos - start));
        if (pos == std::string::npos) break;
        start = pos + 1;
      }
      continue;
    }
    if (std::string(argv[i]) == "--json") { o->json = true; continue; }
    if (std::string(argv[i]) == "--constants") { o->constants = true; continue; }
    if (take_value(argc, argv, i, "device", &v)) {
      if (v != "cpu" && v != "gpu") { fprintf(stderr, "--device must be gpu or cpu\n"); return false; }
      o->cpu = v == "cpu";
      continue;
    }
    if (argv[i][0] == '-') { fprintf(stderr, "Unknown option %s\n", argv[i]); return false; }
    if (!o->lib.empty()) { fprintf(stderr, "Too many positional arguments\n"); return false; }
    o->lib = argv[i];
  }
  if (o->lib.empty()) { fprintf(stderr, "Model Library Path <lib> is required\n"); return false; }
  if (o->gpus < 1) o->gpus = 1;
  return true;
}

struct WorkerResult {
  int32_t ok;
  int32_t runs;
  double avg_ms;      // GPU-event time per run (whole graph call incl. copies)
  double first_ms;    // wall time of the first (warm-up) run
};

// Runs the graph on device `rank` over rows [row0, row0+rows) of dimension 0.
WorkerResult run_worker(const Options &o, int rank, int world, int result_fd) {
  WorkerResult res{0, 0, 0.0, 0.0};
  auto finish = [&](bool ok) {
    res.ok = ok ? 1 : 0;
    if (result_fd >= 0) { ssize_t w = write(result_fd, &res, sizeof(res)); (void)w; }
    return res;
  };
  if (!o.cpu) {
    mgpuSetDefaultDevice(rank);
    mgpuModuleFileLoad(o.ops.c_str());
    gpuOpsInit();
    if (mgpuGetLastError()) return finish(false);
  }

  std::string err;
  ModelInfo *info = ModelInfo::ParseModelInfo(o.input, o.output, o.data, &err);
  if (!info) { fprintf(stderr, "%s\n", err.c_str()); return finish(false); }
  auto params = GetParamsVec(info);
  if (params.empty()) return finish(false);

  // batch shard: rows [row0, row0 + rows) of input 0 / output 0
  const size_t n_out = info->OutputNums();
  size_t row0 = 0, rows = info->GetInputSize(0)[0];
  const size_t total_rows = rows;
  size_t in_row_elems = 1, out_row_elems = 1;
  if (world > 1) {
    if (info->GetOutputSize(0)[0] != total_rows) {
      fprintf(stderr, "--gpus: output 0 and input 0 must share dimension 0\n");
      return finish(false);
    }
    const size_t per = (total_rows + world - 1) / world;
    row0 = per * rank;
    rows = row0 >= total_rows ? 0 : (total_rows - row0 < per ? total_rows - row0 : per);
    in_row_elems = params[n_out]->GetNumElements() / total_rows;
    out_row_elems = info->GetOutputNumElements(0) / total_rows;
    if (rows == 0) { res.runs = 0; return finish(true); }
    // re-describe input 0 as its slice (the data is moved to the front of the buffer) and
    // any rank-1 input of length total_rows (per-sequence lengths) likewise
    FloatTensor *in0 = params[n_out];
    memmove(in0->data(), in0->data() + row0 * in_row_elems, rows * in_row_elems * sizeof(float));
    in0->set_dim0(rows);
    for (size_t i = n_out + 1; i < params.size(); ++i)
      if (params[i]->rank() == 1 && params[i]->shape()[0] == total_rows) {
        memmove(params[i]->data(), params[i]->data() + row0, rows * sizeof(float));
        params[i]->set_dim0(rows);
      }
    params[0]->set_dim0(rows);
  }

  if (o.constants && !o.cpu)
    for (size_t i = n_out + 1; i < params.size(); ++i)
      mgpuRegisterConstant(params[i]->data(), params[i]->GetNumElements() * sizeof(float));

  void *handle = LoadLibrary(o.lib);
  if (!handle) return finish(false);
  RunGraphFuncPtr func = LoadFunc(handle, o.func);
  if (!func) return finish(false);

  const auto t0 = std::chrono::steady_clock::now();
  if (!RunGraphFunc(func, params)) return finish(false);
  res.first_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
  if (!o.cpu && mgpuGetLastError()) return finish(false);

  if (!o.out_data.empty()) {
    if (world == 1) {
      if (!SaveFloatTensor(params, o.out_data)) return finish(false);
    } else {
      // final gather: every worker writes its rows at their offset in the shared file
      const int fd = open(o.out_data.c_str(), O_WRONLY | O_CREAT, 0644);
      if (fd < 0) { perror("open out-data"); return finish(false); }
      const size_t bytes = rows * out_row_elems * sizeof(float);
      const ssize_t put = pwrite(fd, params[0]->data(), bytes, static_cast<off_t>(row0 * out_row_elems * sizeof(float)));
      close(fd);
      if (put != static_cast<ssize_t>(bytes)) return finish(false);
    }
  }

  if (o.rerun > 0 && o.cpu) {
    double elapsed = 0.0;
    for (int i = 0; i < o.rerun; ++i) {
      ClearOutputTensor(info, params);
      const auto b = std::chrono::steady_clock::now();
      RunGraphFunc(func, params);
      elapsed += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - b).count();
    }
    res.runs = o.rerun;
    res.avg_ms = elapsed / o.rerun;
  } else if (o.rerun > 0) {
    mgpu_stream_t stream = mgpuStreamCreate();
    mgpu_event_t begin = mgpuEventEnableTimeCreate(), end = mgpuEventEnableTimeCreate();
    double elapsed = 0.0;
    for (int i = 0; i < o.rerun; ++i) {
      ClearOutputTensor(info, params);
      mgpuEventRecord(begin, stream);
      RunGraphFunc(func, params);
      mgpuEventRecord(end, stream);
      mgpuEventSynchronize(end);
      elapsed += mgpuEventElapsedTime(begin, end);
    }
    mgpuEventDestroy(begin);
    mgpuEventDestroy(end);
    mgpuStreamDestroy(stream);
    res.runs = o.rerun;
    res.avg_ms = elapsed / o.rerun;
  }
  bool ok = true;
  if (!o.cpu) {
    ok = mgpuGetLastError() == 0 && mgpuOpsCheckDeviceStatus(nullptr) == 0;
    gpuOpsDeinit();
    mgpuModuleUnload();
  }
  for (auto *p : params) delete p;
  delete info;
  return finish(ok);
}

}  // namespace

int main(int argc, char **argv) {
  // A lowered graph mallocs its result on every call and the runner frees it.  Keep such
  // blocks in the heap instead of mapping and unmapping them, so that only the first call
  // pays the page faults (33.5 MB of output = 8192 faults per call otherwise).
  mallopt(M_MMAP_THRESHOLD, 1 << 30);
  mallopt(M_TRIM_THRESHOLD, 1 << 30);
  Options o;
  if (!parse(argc, argv, &o)) {
    fprintf(stderr, "Failed to parse options\n");
    return 1;
  }

  if (o.gpus == 1) {
    WorkerResult r = run_worker(o, 0, 1, -1);
    if (!r.ok) {
      fprintf(stderr, "multi-device-gpu-runner: failed: %s\n", mgpuGetLastErrorString());
      return 1;
    }
    if (o.rerun) {
      printf("Run \t%d\ttimes\n", r.runs);
      printf("Average time:\t%g\tseconds\n", r.avg_ms / 1000.0);
    }
    if (o.json) printf("{\"gpus\": 1, \"runs\": %d, \"avg_ms\": %.6f, \"first_ms\": %.3f}\n", r.runs, r.avg_ms, r.first_ms);
    return 0;
  }

  // One worker process per GPU.  The parent never touches CUDA; it supervises the workers
  // with a deadline and reports any that died, failed or ran out of time.
  if (!o.out_data.empty()) {
    const int fd = open(o.out_data.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (fd >= 0) close(fd);
  }
  struct Child { pid_t pid; int fd; bool done; WorkerResult r; };
  std::vector<Child> kids;
  for (int rank = 0; rank < o.gpus; ++rank) {
    int pipefd[2];
    if (pipe(pipefd) != 0) { perror("pipe"); return 1; }
    const pid_t pid = fork();
    if (pid < 0) { perror("fork"); return 1; }
    if (pid == 0) {
      close(pipefd[0]);
      WorkerResult r = run_worker(o, rank, o.gpus, pipefd[1]);
      close(pipefd[1]);
      _exit(r.ok ? 0 : 2);
    }
    close(pipefd[1]);
    kids.push_back(Child{pid, pipefd[0], false, WorkerResult{0, 0, 0.0, 0.0}});
  }
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(o.timeout_s);
  int failures = 0;
  size_t remaining = kids.size();
  while (remaining > 0) {
    bool progressed = false;
    for (size_t i = 0; i < kids.size(); ++i) {
      Child &c = kids[i];
      if (c.done) continue;
      int status = 0;
      const pid_t w = waitpid(c.pid, &status, WNOHANG);
      if (w == c.pid) {
        c.done = true;
        --remaining;
        progressed = true;
        const ssize_t got = read(c.fd, &c.r, sizeof(c.r));
        close(c.fd);
        const bool ok = WIFEXITED(status) && WEXITSTATUS(status) == 0 && got == static_cast<ssize_t>(sizeof(c.r)) && c.r.ok;
        if (!ok) {
          ++failures;
          if (WIFSIGNALED(status)) fprintf(stderr, "worker %zu died with signal %d\n", i, WTERMSIG(status));
          else fprintf(stderr, "worker %zu failed (exit %d)\n", i, WIFEXITED(status) ? WEXITSTATUS(status) : -1);
        }
      }
    }
    if (remaining == 0) break;
    if (std::chrono::steady_clock::now() > deadline) {
      for (Child &c : kids)
        if (!c.done) {
          fprintf(stderr, "worker pid %d exceeded the %d s deadline\n", static_cast<int>(c.pid), o.timeout_s);
          kill(c.pid, SIGKILL);
          waitpid(c.pid, nullptr, 0);
          close(c.fd);
          c.done = true;
          ++failures;
        }
      break;
    }
    if (!progressed) usleep(2000);
  }
  if (failures) {
    fprintf(stderr, "multi-device-gpu-runner: %d of %d workers failed\n", failures, o.gpus);
    return 1;
  }
  double worst = 0.0;
  for (const Child &c : kids) worst = c.r.avg_ms > worst ? c.r.avg_ms : worst;
  if (o.rerun) {
    printf("Run \t%d\ttimes on %d GPUs\n", o.rerun, o.gpus);
    printf("Average time:\t%g\tseconds (slowest worker)\n", worst / 1000.0);
  }
  if (o.json) printf("{\"gpus\": %d, \"runs\": %d, \"avg_ms\": %.6f}\n", o.gpus, o.rerun, worst);
  return 0;
}
