// Dense comparison in the reference's convention (spmm/utils/compare.cpp:2-28): both operands
// are brought to the host, the maximum ABSOLUTE error is compared with 0.1, and ktype == "div"
// divides the first operand by EXE_NUM_CUDA to undo the reference's 200 accumulating launches
// (never needed with this library's LBSpMM, kept for callers that compare against a run of the
// reference).  Returns the error instead of aborting; the position reported is the arg-max
// (the reference always reports the last index, compare.cpp:19).
#pragma once
#include <cmath>
#include <iostream>
#include <string>

#include "spmm/utils/timer_cuda.h"
#include "starml/basic/matrix.h"

inline double ExpectEqualDenseWithError(const starml::Matrix& mat1, const starml::Matrix& mat2,
                                        const std::string& ktype = "", double threshold = 0.1) {
  if (mat1.size() != mat2.size() || mat1.ndims() != mat2.ndims())
    throw hpspmm::Error(HPSPMM_ERR_INVALID, "compare: shapes differ");
  const starml::Matrix a = mat1.to(starml::kCPU), b = mat2.to(starml::kCPU);
  const float* pa = a.data<float>();
  const float* pb = b.data<float>();
  double err_max = 0.0;
  int64_t pos = -1;
  for (int64_t i = 0; i < a.size(); ++i) {
    const float x = ktype == "div" ? pa[i] / (float)EXE_NUM_CUDA : pa[i];
    const double e = std::fabs((double)x - (double)pb[i]);
    if (e > err_max) {
      err_max = e;
      pos = i;
    }
  }
  if (err_max < threshold)
    std::cout << "PASSed!! max_err = " << err_max << " < " << threshold << std::endl;
  else
    std::cout << "Wrong!! max_err = " << err_max << " >= " << threshold << " at pos: " << pos << std::endl;
  return err_max;
}
