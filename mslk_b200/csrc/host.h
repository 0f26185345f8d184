// Host-side helpers shared by the launchers: error reporting, the per-device
// status word, SM count and TMA descriptor encoding.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MSLK_API extern "C" __attribute__((visibility("default")))

namespace mslk_b200 {

// Records `msg` (printf-style) as the calling thread's last error and returns `code`.
int fail(int code, const char *fmt, ...);
void clear_error();

// Returns 0 on success (after recording nothing) or records the CUDA error string.
int check_cuda(cudaError_t e, const char *what);

// Device pointer of the status word of the current device (nullptr on failure, error recorded).
int *device_status_ptr();

// Number of SMs of the current device (cached per device).
int sm_count();

// Programmatic dependent launch: fills `attr` with the stream-serialization attribute and returns 1 when the
// launchers should use it (default), 0 when the environment variable MSLK_B200_PDL=0 switched it off (read once).
int pdl_attribute(cudaLaunchAttribute *attr);

// Encodes a 2-D row-major tensor map: `rows` x `cols_bytes` bytes-per-row view of
// `base` with row pitch `pitch_bytes`, box {box_cols_bytes, box_rows}, 1-byte
// elements, the given swizzle, zero fill out of bounds.  Returns 0 or records an error.
int make_tmap_2d_bytes(CUtensorMap *out, const void *base, uint64_t cols_bytes, uint64_t rows,
                       uint64_t pitch_bytes, uint32_t box_cols_bytes, uint32_t box_rows,
                       CUtensorMapSwizzle swizzle);

// Same for 2-byte (bf16) elements: cols / box_cols are element counts.
// 2-D map over 32-bit words, no swizzle (rows wider than 256 bytes, e.g. 512-byte scale atoms)
int make_tmap_2d_u32(CUtensorMap *out, const void *base, uint64_t cols, uint64_t rows, uint64_t pitch_bytes,
                     uint32_t box_cols, uint32_t box_rows);
int make_tmap_2d_bf16(CUtensorMap *out, const void *base, uint64_t cols, uint64_t rows, uint64_t pitch_bytes,
                      uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle swizzle);

}  // namespace mslk_b200
