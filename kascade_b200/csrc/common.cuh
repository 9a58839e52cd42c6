// Shared host/device helpers of libkascade_b200.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "kascade_b200.h"

namespace kb200 {

// thread-local error text returned by kb200_last_error()
void set_error(const char* fmt, ...);
bool initialised(int* device_out);
int check_on_current_device(const void* ptr, const char* what);

#define KB_ENTRY(first_ptr, what)                                                                 \
  do {                                                                                            \
    KB_REQUIRE(kb200::initialised(nullptr),                                                       \
               "kb200_init has not been called for the device that is current in this thread");  \
    if (kb200::check_on_current_device(first_ptr, what) != 0) return -1;                          \
  } while (0)

#define KB_REQUIRE(cond, ...)        \
  do {                               \
    if (!(cond)) {                   \
      kb200::set_error(__VA_ARGS__); \
      return -1;                     \
    }                                \
  } while (0)

#define KB_CUDA(expr)                                                            \
  do {                                                                           \
    cudaError_t e__ = (expr);                                                    \
    if (e__ != cudaSuccess) {                                                    \
      kb200::set_error("%s failed: %s", #expr, cudaGetErrorString(e__));         \
      return -1;                                                                 \
    }                                                                            \
  } while (0)

#define KB_CHECK_LAUNCH(name)                                                    \
  do {                                                                           \
    cudaError_t e__ = cudaGetLastError();                                        \
    if (e__ != cudaSuccess) {                                                    \
      kb200::set_error("launch of %s failed: %s", name, cudaGetErrorString(e__)); \
      return -1;                                                                 \
    }                                                                            \
  } while (0)

constexpr int kD = KB200_HEAD_DIM;       // head dimension
constexpr int kHg = KB200_GROUP_SIZE;    // query heads per KV head
constexpr int kTile = KB200_TILE;        // queries per prefill tile
constexpr float kLog2e = 1.4426950408889634f;

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

int sm_count();

// per-module init hooks (raise dynamic shared memory limits); defined in the kernel files
int init_decode();
int init_prefill();
int init_selftest();

}  // namespace kb200
