// Host-side runner plumbing: model shape flags, MLIR memref descriptors for fp32 tensors,
// raw little-endian fp32 files, dlopen / dlsym of a lowered model library and the variadic
// call of its entry point.  Same roles and function names as the reference's
// lib/Runtime/{ModelInfo,RuntimeUtil}.cpp and Runtime/TensorDescripter.h, written without
// the LLVM support library.
//
// A lowered graph is entered through
//     void _mlir_ciface_main_graph(OutDesc*..., InDesc*...)
// (doc/runtime.md:7-9): output descriptors first, then inputs.  A descriptor of rank N is
//     { float* allocated; float* aligned; intptr_t offset; intptr_t sizes[N]; intptr_t strides[N]; }
// (Runtime/TensorDescripter.h:9-14).  The callee mallocs the output buffer and fills the
// descriptor; the caller frees it.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace multi_device {

// A rank-erased memref descriptor: 3 + 2*rank machine words laid out exactly like the
// templated struct above, so its address can be passed to a lowered graph.
class FloatTensor {
public:
  explicit FloatTensor(const std::vector<size_t> &shape);
  ~FloatTensor();
  FloatTensor(const FloatTensor &) = delete;
  FloatTensor &operator=(const FloatTensor &) = delete;

  void *descriptor() { return words_.data(); }
  size_t rank() const { return shape_.size(); }
  const std::vector<size_t> &shape() const { return shape_; }
  size_t GetNumElements() const;
  float *data() const { return reinterpret_cast<float *>(words_[1]); }
  // 64-byte aligned zero-initialised buffer owned by the tensor (TensorDescripter.h:43-52)
  void InitData();
  // adopt a malloc-family buffer (TensorDescripter.h:54-57)
  void InitData(float *data);
  // frees the buffer the descriptor points at (also one a callee malloc'd) and nulls it
  void clear();
  // re-describe the tensor with a different extent of dimension 0 (batch sharding)
  void set_dim0(size_t n);

private:
  std::vector<size_t> shape_;
  std::vector<intptr_t> words_;
};

// "--input 3_640_640,3_640_640 --output 3_640_640 --data a.dat,b.dat" (ModelInfo.cpp:13-28)
struct ModelInfo {
  static ModelInfo *ParseModelInfo(const std::string &inputs, const std::string &outputs,
                                   const std::vector<std::string> &data_files, std::string *error);
  size_t InputNums() const { return inputSizes.size(); }
  size_t OutputNums() const { return outputSizes.size(); }
  size_t GetInputNumElements(int idx) const;
  size_t GetOutputNumElements(int idx) const;
  std::vector<size_t> &GetInputSize(int idx) { return inputSizes[idx]; }
  std::vector<size_t> &GetOutputSize(int idx) { return outputSizes[idx]; }
  std::string GetFile(int idx) const { return inputData[idx]; }
  bool ExistFile() const { return !inputData.empty(); }

  std::vector<std::vector<size_t>> inputSizes, outputSizes;
  std::vector<std::string> inputData;
};

// "3_640_640" -> {3,640,640}; "a_b,c" -> {{a,b},{c}}.  Throws std::invalid_argument on
// anything that is not a positive integer.
std::vector<size_t> ParseOneShape(const std::string &text);
std::vector<std::vector<size_t>> ParseShapes(const std::string &text);

typedef void (*RunGraphFuncPtr)(...);

// nullptr (and a message on stderr) if the file is missing or shorter than numElements floats
float *LoadFloatData(const std::string &file, size_t numElements);
bool SaveFloatData(const std::string &file, const float *data, size_t numElements);
// output 0 -> raw fp32 file (RuntimeUtil.cpp:54-75)
bool SaveFloatTensor(std::vector<FloatTensor *> &params, const std::string &file);
// outputs first (no buffer), then inputs (from files, or zero-filled) (RuntimeUtil.cpp:100-112)
std::vector<FloatTensor *> GetParamsVec(ModelInfo *info);
void *LoadLibrary(const std::string &libName);
RunGraphFuncPtr LoadFunc(void *handle, const std::string &funcName);
// up to 16 descriptors (the reference stops at 5, RuntimeUtil.cpp:133-157)
bool RunGraphFunc(RunGraphFuncPtr func, std::vector<FloatTensor *> &params);
void ClearOutputTensor(ModelInfo *info, std::vector<FloatTensor *> &params);

}  // namespace multi_device
