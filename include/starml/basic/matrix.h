// Minimal stand-in for the reference's starml tensor layer, sized for the SpMM path only.
//
// The reference's `starml::Matrix` (include/starml/basic/matrix.h:14-77) is a ref-counted typed
// buffer on CPU or CUDA with allocator / handle registries and a dispatcher behind it.  Callers
// of the SpMM path use a small part of that surface: construction from a shape, `dim`, `size`,
// `data<T>()`, `mutable_data<T>()`, `to(device)`, and the `full` / `rand` / `empty` factories.
// This header provides exactly that part, header-only, on top of the C ABI in hpspmm.h
// (device memory and copies go through hpspmm_dev_alloc / hpspmm_memcpy_*).  Errors are
// exceptions (`hpspmm::Error`) rather than the reference's log-and-abort.
#pragma once
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <typeinfo>
#include <vector>

#include "hpspmm.h"

namespace hpspmm {

class Error : public std::runtime_error {
 public:
  Error(int status, const std::string& what) : std::runtime_error(what), status_(status) {}
  int status() const { return status_; }

 private:
  int status_;
};

// One lazily created context per device ordinal for the wrappers.
inline hpspmm_ctx* context(int device = 0) {
  static hpspmm_ctx* ctxs[64] = {nullptr};
  if (device < 0 || device >= 64) throw Error(HPSPMM_ERR_INVALID, "device ordinal out of range");
  if (!ctxs[device]) {
    const int st = hpspmm_ctx_create(device, &ctxs[device]);
    if (st != HPSPMM_OK) throw Error(st, std::string("hpspmm_ctx_create: ") + hpspmm_status_string(st));
  }
  return ctxs[device];
}

inline void check(int st, const char* what, int device = 0) {
  if (st == HPSPMM_OK) return;
  std::string msg = std::string(what) + ": " + hpspmm_status_string(st);
  const char* detail = hpspmm_last_error(context(device));
  if (detail && detail[0]) msg += std::string(" (") + detail + ")";
  throw Error(st, msg);
}

}  // namespace hpspmm

namespace starml {

enum class DeviceType : int { CPU = 0, CUDA = 1 };
constexpr DeviceType kCPU = DeviceType::CPU;
constexpr DeviceType kCUDA = DeviceType::CUDA;

class Device {
 public:
  Device(DeviceType type = kCPU, int index = 0) : type_(type), index_(index) {}
  DeviceType type() const { return type_; }
  int index() const { return index_; }
  bool operator==(const Device& o) const { return type_ == o.type_ && index_ == o.index_; }

 private:
  DeviceType type_;
  int index_;
};

enum class DataTypeKind : int { Int32 = 0, Int64 = 1, Float = 2, Double = 3 };
constexpr DataTypeKind kInt32 = DataTypeKind::Int32;
constexpr DataTypeKind kInt64 = DataTypeKind::Int64;
constexpr DataTypeKind kFloat = DataTypeKind::Float;
constexpr DataTypeKind kDouble = DataTypeKind::Double;

class DataType {
 public:
  DataType(DataTypeKind kind = kFloat) : kind_(kind) {}
  DataTypeKind type() const { return kind_; }
  size_t size() const { return (kind_ == kInt32 || kind_ == kFloat) ? 4 : 8; }
  template <typename T>
  bool is_valid() const {
    switch (kind_) {
      case kInt32: return std::is_integral<T>::value && sizeof(T) == 4;
      case kInt64: return std::is_integral<T>::value && sizeof(T) == 8;
      case kFloat: return std::is_same<T, float>::value;
      default: return std::is_same<T, double>::value;
    }
  }

 private:
  DataTypeKind kind_;
};

using Shape = std::vector<int64_t>;

class Matrix {
 public:
  Matrix() : size_(0) {}
  Matrix(const Shape& shape, const Device& device, const DataType& data_type)
      : shape_(shape), device_(device), dtype_(data_type) {
    size_ = 1;
    for (int64_t d : shape_) {
      if (d < 0) throw hpspmm::Error(HPSPMM_ERR_INVALID, "negative dimension");
      size_ *= d;
    }
    allocate();
  }
  Matrix(const Shape& shape, const DataType& data_type, const Device& device)
      : Matrix(shape, device, data_type) {}

  // 64-bit on purpose: the reference's int size overflows at N*K = 2^31 (matrix.h:71)
  int64_t size() const { return size_; }
  const Shape& dims() const { return shape_; }
  int64_t dim(int axis) const { return shape_.at((size_t)axis); }
  int ndims() const { return (int)shape_.size(); }
  const Device& device() const { return device_; }
  const DataType& data_type() const { return dtype_; }
  bool is_cuda() const { return device_.type() == kCUDA; }
  const void* raw_data() const { return data_.get(); }
  void* raw_mutable_data() const { return data_.get(); }
  size_t nbytes() const { return (size_t)size_ * dtype_.size(); }

  template <typename T>
  const T* data() const {
    require_type<T>();
    return static_cast<const T*>(data_.get());
  }
  template <typename T>
  T* mutable_data() const {
    require_type<T>();
    return static_cast<T*>(data_.get());
  }

  // Deep copy onto another device (the reference's Matrix::to, spmm/starml/basic/matrix.cpp:42-44).
  // Unlike the reference, CUDA -> CUDA really copies (its device-to-device kernel is an empty
  // stub, spmm/starml/operators/cuda/copy_kernel.cu:43-44).
  Matrix to(Device new_device) const {
    Matrix out(shape_, new_device, dtype_);
    if (size_ == 0) return out;
    const int dev = is_cuda() ? device_.index() : new_device.index();
    hpspmm_ctx* ctx = (is_cuda() || out.is_cuda()) ? hpspmm::context(dev) : nullptr;
    if (!is_cuda() && !out.is_cuda()) {
      std::memcpy(out.data_.get(), data_.get(), nbytes());
    } else if (!is_cuda()) {
      hpspmm::check(hpspmm_memcpy_h2d(ctx, out.data_.get(), data_.get(), nbytes(), nullptr), "h2d", dev);
      hpspmm::check(hpspmm_stream_sync(ctx, nullptr), "sync", dev);
    } else if (!out.is_cuda()) {
      hpspmm::check(hpspmm_memcpy_d2h(ctx, out.data_.get(), data_.get(), nbytes(), nullptr), "d2h", dev);
      hpspmm::check(hpspmm_stream_sync(ctx, nullptr), "sync", dev);
    } else {
      hpspmm::check(hpspmm_memcpy_d2d(ctx, out.data_.get(), data_.get(), nbytes(), nullptr), "d2d", dev);
      hpspmm::check(hpspmm_stream_sync(ctx, nullptr), "sync", dev);
    }
    return out;
  }
  Matrix to(DeviceType t) const { return to(Device(t, 0)); }

 private:
  template <typename T>
  void require_type() const {
    if (!dtype_.is_valid<T>())
      throw hpspmm::Error(HPSPMM_ERR_INVALID, std::string("Matrix holds another element type than ") + typeid(T).name());
  }
  void allocate() {
    if (size_ == 0) return;
    if (device_.type() == kCPU) {
      void* p = std::malloc(nbytes());
      if (!p) throw hpspmm::Error(HPSPMM_ERR_OOM, "host allocation failed");
      data_ = std::shared_ptr<void>(p, std::free);
    } else {
      const int dev = device_.index();
      hpspmm_ctx* ctx = hpspmm::context(dev);
      void* p = nullptr;
      hpspmm::check(hpspmm_dev_alloc(ctx, nbytes(), &p), "hpspmm_dev_alloc", dev);
      data_ = std::shared_ptr<void>(p, [ctx](void* q) { hpspmm_dev_free(ctx, q); });
    }
  }

  int64_t size_;
  Shape shape_;
  Device device_;
  DataType dtype_;
  std::shared_ptr<void> data_;
};

}  // namespace starml
