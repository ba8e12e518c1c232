// `full`, `rand`, `empty` for the SpMM path (reference: include/starml/operators/factories.h,
// spmm/starml/operators/cpu/factories_kernel.cpp:5-28, cuda/factories_kernel.cu:8-17).
// `rand` is SEEDED here: element i is a pure function of (seed, stream, i), on host and device
// alike; the reference draws from an unseeded std::random_device and supports the CPU only.
#pragma once
#include "starml/basic/matrix.h"

namespace starml {

inline Matrix empty(const Shape& shape, const Device& device, const DataType& data_type) {
  return Matrix(shape, device, data_type);
}

inline Matrix full(const Shape& shape, const Device& device, const DataType& data_type, double init_val) {
  Matrix m(shape, device, data_type);
  if (m.size() == 0) return m;
  if (device.type() == kCPU) {
    if (data_type.type() == kFloat) {
      float* p = m.mutable_data<float>();
      for (int64_t i = 0; i < m.size(); ++i) p[i] = (float)init_val;
    } else if (data_type.type() == kInt32) {
      int32_t* p = m.mutable_data<int32_t>();
      for (int64_t i = 0; i < m.size(); ++i) p[i] = (int32_t)init_val;
    } else {
      throw hpspmm::Error(HPSPMM_ERR_UNSUPPORTED, "full: only Float and Int32 on this path");
    }
  } else {
    hpspmm_ctx* ctx = hpspmm::context(device.index());
    if (data_type.type() == kFloat) {
      hpspmm::check(hpspmm_fill_f32(ctx, m.mutable_data<float>(), m.size(), (float)init_val, nullptr), "fill");
    } else if (init_val == 0.0) {
      hpspmm::check(hpspmm_memset(ctx, m.raw_mutable_data(), 0, m.nbytes(), nullptr), "memset");
    } else {
      throw hpspmm::Error(HPSPMM_ERR_UNSUPPORTED, "full: non-zero integer fill on the device");
    }
    hpspmm::check(hpspmm_stream_sync(ctx, nullptr), "sync");
  }
  return m;
}

inline Matrix rand(const Shape& shape, const Device& device, const DataType& data_type, double start,
                   double end, uint64_t seed = 1, uint64_t stream = 100) {
  if (data_type.type() != kFloat) throw hpspmm::Error(HPSPMM_ERR_UNSUPPORTED, "rand: Float only");
  Matrix m(shape, device, data_type);
  if (m.size() == 0) return m;
  if (device.type() == kCPU) {
    hpspmm::check(hpspmm_host_fill_uniform_f32(m.mutable_data<float>(), m.size(), seed, stream,
                                               (float)start, (float)end), "host_fill_uniform");
  } else {
    hpspmm_ctx* ctx = hpspmm::context(device.index());
    hpspmm::check(hpspmm_fill_uniform_f32(ctx, m.mutable_data<float>(), m.size(), seed, stream,
                                          (float)start, (float)end, nullptr), "fill_uniform");
    hpspmm::check(hpspmm_stream_sync(ctx, nullptr), "sync");
  }
  return m;
}

}  // namespace starml
