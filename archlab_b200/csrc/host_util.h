// Host-side helpers shared by the launchers: TMA descriptor construction through the driver entry
// point (no link-time dependency on libcuda), the launch counter, and error plumbing.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nga {

// Build a rank-3 tiled tensor map over a bf16 / fp32 / uint8 array.
//   dims    = {inner, rows, batch} extents in elements
//   strides = {row stride, batch stride} in BYTES (multiples of 16)
//   box     = {inner, rows, 1} tile extents in elements; swizzle128 selects the 128-byte swizzle
// Returns 0 on success.
int make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes,
                 uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                 uint64_t stride2_bytes, uint32_t b0, uint32_t b1, bool swizzle128);

void count_launch();
int sm_count();
int current_device_slot();   // cudaGetDevice() clamped to [0, kMaxDevices)

// Function attributes (the opt-in to more than 48 KB of dynamic shared memory, occupancy results)
// belong to a device, not to the process: one slot per device, indexed by the CURRENT device, so a
// process that drives several GPUs sets them up on each.  The caller's buffers and stream must
// belong to the current device.
constexpr int kMaxDevices = 64;
template <typename T>
struct PerDevice {
  T v[kMaxDevices] = {};
  T& here() { return v[current_device_slot()]; }
};

#define NGA_CHECK_LAUNCH()                              \
  do {                                                  \
    cudaError_t e__ = cudaGetLastError();               \
    if (e__ != cudaSuccess) return -1000 - (int)e__;    \
  } while (0)

}  // namespace nga
