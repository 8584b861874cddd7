#include "host_runtime.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <dlfcn.h>
#include <stdexcept>

namespace multi_device {

FloatTensor::FloatTensor(const std::vector<size_t> &shape) : shape_(shape), words_(3 + 2 * shape.size(), 0) {
  set_dim0(shape.empty() ? 0 : shape[0]);
}

void FloatTensor::set_dim0(size_t n) {
  const size_t r = shape_.size();
  if (r == 0) return;
  shape_[0] = n;
  intptr_t stride = 1;
  for (size_t i = r; i-- > 0;) {
    words_[3 + i] = static_cast<intptr_t>(shape_[i]);
    words_[3 + r + i] = stride;
    stride *= static_cast<intptr_t>(shape_[i]);
  }
}

FloatTensor::~FloatTensor() { clear(); }

size_t FloatTensor::GetNumElements() const {
  size_t n = 1;
  for (size_t s : shape_) n *= s;
  return n;
}

void FloatTensor::InitData() {
  clear();
  size_t bytes = GetNumElements() * sizeof(float);
  bytes = (bytes + 63) / 64 * 64;
  float *p = static_cast<float *>(aligned_alloc(64, bytes ? bytes : 64));
  if (p) memset(p, 0, bytes ? bytes : 64);
  InitData(p);
}

void FloatTensor::InitData(float *data) {
  words_[0] = reinterpret_cast<intptr_t>(data);
  words_[1] = reinterpret_cast<intptr_t>(data);
}

void FloatTensor::clear() {
  if (words_[0]) free(reinterpret_cast<void *>(words_[0]));
  words_[0] = words_[1] = 0;
}

std::vector<size_t> ParseOneShape(const std::string &text) {
  std::vector<size_t> shape;
  size_t start = 0;
  while (true) {
    const size_t pos = text.find('_', start);
    const std::string tok = text.substr(start, pos == std::string::npos ? std::string::npos : pos - start);
    if (tok.empty() || tok.find_first_not_of("0123456789") != std::string::npos)
      throw std::invalid_argument("bad shape '" + text + "'");
    const unsigned long v = std::stoul(tok);
    if (v == 0) throw std::invalid_argument("zero extent in shape '" + text + "'");
    shape.push_back(v);
    if (pos == std::string::npos) break;
    start = pos + 1;
  }
  return shape;
}

std::vector<std::vector<size_t>> ParseShapes(const std::string &text) {
  std::vector<std::vector<size_t>> shapes;
  size_t start = 0;
  while (true) {
    const size_t pos = text.find(',', start);
    shapes.push_back(ParseOneShape(text.substr(start, pos == std::string::npos ? std::string::npos : pos - start)));
    if (pos == std::string::npos) break;
    start = pos + 1;
  }
  return shapes;
}

ModelInfo *ModelInfo::ParseModelInfo(const std::string &inputs, const std::string &outputs,
                                     const std::vector<std::string> &data_files, std::string *error) {
  ModelInfo *info = new ModelInfo();
  try {
    info->inputSizes = ParseShapes(inputs);
    info->outputSizes = ParseShapes(outputs);
  } catch (const std::exception &e) {
    if (error) *error = e.what();
    delete info;
    return nullptr;
  }
  for (auto &s : info->inputSizes)
    if (s.size() > 4) { if (error) *error = "Not support dim greater than 4."; delete info; return nullptr; }
  for (auto &s : info->outputSizes)
    if (s.size() > 4) { if (error) *error = "Not support dim greater than 4."; delete info; return nullptr; }
  info->inputData = data_files;
  if (!info->inputData.empty() && info->inputData.size() != info->InputNums()) {
    if (error) *error = "Data num not equal input num!";
    delete info;
    return nullptr;
  }
  return info;
}

size_t ModelInfo::GetInputNumElements(int idx) const {
  size_t n = 1;
  for (size_t s : inputSizes[idx]) n *= s;
  return n;
}
size_t ModelInfo::GetOutputNumElements(int idx) const {
  size_t n = 1;
  for (size_t s : outputSizes[idx]) n *= s;
  return n;
}

float *LoadFloatData(const std::string &file, size_t numElements) {
  FILE *f = fopen(file.c_str(), "rb");
  if (!f) {
    fprintf(stderr, "Error reading file: %s\n", file.c_str());
    return nullptr;
  }
  size_t bytes = numElements * sizeof(float);
  float *data = static_cast<float *>(aligned_alloc(64, (bytes + 63) / 64 * 64 + 64));
  const size_t got = data ? fread(data, sizeof(float), numElements, f) : 0;
  fclose(f);
  if (got < numElements) {
    fprintf(stderr, "Wrong File size\n");
    free(data);
    return nullptr;
  }
  return data;
}

bool SaveFloatData(const std::string &file, const float *data, size_t numElements) {
  FILE *f = fopen(file.c_str(), "wb");
  if (!f) {
    fprintf(stderr, "Error open file to write: %s\n", file.c_str());
    return false;
  }
  const size_t put = fwrite(data, sizeof(float), numElements, f);
  fclose(f);
  return put == numElements;
}

bool SaveFloatTensor(std::vector<FloatTensor *> &params, const std::string &file) {
  if (params.empty() || !params[0]->data()) return false;
  return SaveFloatData(file, params[0]->data(), params[0]->GetNumElements());
}

std::vector<FloatTensor *> GetParamsVec(ModelInfo *info) {
  std::vector<FloatTensor *> params;
  for (size_t i = 0; i < info->OutputNums(); ++i) params.push_back(new FloatTensor(info->GetOutputSize(i)));
  for (size_t i = 0; i < info->InputNums(); ++i) {
    FloatTensor *t = new FloatTensor(info->GetInputSize(i));
    if (info->ExistFile()) {
      float *d = LoadFloatData(info->GetFile(i), t->GetNumElements());
      if (!d) {
        for (auto *p : params) delete p;
        delete t;
        return {};
      }
      t->InitData(d);
    } else {
      t->InitData();
    }
    params.push_back(t);
  }
  return params;
}

void *LoadLibrary(const std::string &libName) {
  void *handle = dlopen(libName.c_str(), RTLD_LAZY);
  if (!handle) fprintf(stderr, "Failed to open library:%s\n", dlerror());
  return handle;
}

RunGraphFuncPtr LoadFunc(void *handle, const std::string &funcName) {
  dlerror();
  RunGraphFuncPtr func = reinterpret_cast<RunGraphFuncPtr>(dlsym(handle, funcName.c_str()));
  const char *err = dlerror();
  if (err || !func) {
    fprintf(stderr, "Failed to find run function: %s\n", err ? err : funcName.c_str());
    return nullptr;
  }
  return func;
}

bool RunGraphFunc(RunGraphFuncPtr func, std::vector<FloatTensor *> &params) {
  void *p[16] = {nullptr};
  if (params.size() > 16) {
    fprintf(stderr, "Not Support params more than 16.\n");
    return false;
  }
  for (size_t i = 0; i < params.size(); ++i) p[i] = params[i]->descriptor();
  switch (params.size()) {
  case 0: func(); break;
  case 1: func(p[0]); break;
  case 2: func(p[0], p[1]); break;
  case 3: func(p[0], p[1], p[2]); break;
  case 4: func(p[0], p[1], p[2], p[3]); break;
  case 5: func(p[0], p[1], p[2], p[3], p[4]); break;
  case 6: func(p[0], p[1], p[2], p[3], p[4], p[5]); break;
  case 7: func(p[0], p[1], p[2], p[3], p[4], p[5], p[6]); break;
  case 8: func(p[0], p[1], p[2], p[3], p[4], p[5], p[6], p[7]); break;
  default:
    func(p[0], p[1], p[2], p[3], p[4], p[5], p[6], p[7], p[8], p[9], p[10], p[11], p[12], p[13], p[14], p[15]);
    break;
  }
  return true;
}

void ClearOutputTensor(ModelInfo *info, std::vector<FloatTensor *> &params) {
  for (size_t i = 0; i < info->OutputNums() && i < params.size(); ++i) params[i]->clear();
}

}  // namespace multi_device
