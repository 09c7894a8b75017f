// Host-side helpers shared by the launchers: error reporting, TMA descriptor creation, the device
// status word.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/fa_b200.h"

namespace fa {

// Records the message returned by fa_last_error() for the calling thread and returns `code`.
int set_error(int code, const std::string& msg);
const std::string& last_error();

#define FA_CHECK_ARG(cond, msg)                                             \
  do {                                                                      \
    if (!(cond)) return ::fa::set_error(FA_ERR_INVALID_ARGUMENT, (msg));    \
  } while (0)

#define FA_CHECK_CUDA(expr)                                                              \
  do {                                                                                   \
    cudaError_t err__ = (expr);                                                          \
    if (err__ != cudaSuccess)                                                            \
      return ::fa::set_error(FA_ERR_CUDA, std::string(#expr) + ": " +                    \
                                              cudaGetErrorString(err__));                \
  } while (0)

// Encodes a rank-4 fp16 tensor map (dims innermost first) with a {64, 1, box_rows, 1} box and the
// 128-byte swizzle.  dims = {d, heads, rows, batch}; strides in elements for heads, rows, batch.
// Returns 0 or a negative FA_ERR_* code (message recorded).
int make_tensor_map_4d(CUtensorMap* map, const void* base, int d, int64_t heads, int64_t rows,
                       int64_t batch, int64_t head_stride, int64_t row_stride, int64_t batch_stride,
                       int box_rows, const char* what);

// Checks that the current device is an sm_100 part; caches the answer per device.
int check_device_sm100();

// Address of the per-device status word kernels write when a bounded wait gives up.
int* device_status_ptr();

// Work counters of the persistent kernels: a pool of {next item, finished CTAs} pairs in device memory, all zero
// between launches (the last CTA of a launch to finish puts its pair back to zero).  Every launch takes the next
// pair of the pool in turn, so launches that overlap on different streams do not share one unless kSchedSlots
// launches lie between them.  fa_device_status(1) clears the pool together with a non-zero status word (a
// launch that gave up on a wait leaves its pair dirty).
constexpr int kSchedSlots = 1024;
int* next_sched_slot();

// Number of SMs of the current device (cached); 0 on error.
int device_sm_count();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace fa
