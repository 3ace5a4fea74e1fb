// Helpers shared by the translation units of the library's host layer.
#pragma once
#include <cuda_runtime.h>

#include "../../include/walk_b200.h"

namespace walk_b200 {
namespace host {

// Records a printf-style message as the calling thread's last error and returns `code`.
int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
// Checks cudaGetLastError() after a launch; counts the launch when it succeeded.
int check_launch(const char* what);
// Multiprocessor count of the current device (cached per device).
int sm_count();

}  // namespace host
}  // namespace walk_b200

#define WALK_CUDA_TRY(expr)                                                                              \
  do {                                                                                                   \
    cudaError_t err__ = (expr);                                                                          \
    if (err__ != cudaSuccess)                                                                            \
      return ::walk_b200::host::fail(WALK_B200_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__)); \
  } while (0)
