// Allocation-free entry point of the native library.
//
// This entry point has no counterpart in the reference (LLNL/lbann): there every
// reduction workspace is a matrix owned by the layer object.  It exists for callers that
// must not touch the device allocator (for instance inside a region where allocation is
// forbidden or would synchronise): the per-column reduction below keeps its workspace in a
// fixed array inside the library image instead of a buffer passed in by the caller.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest number of columns the built-in workspace serves (2 x 4096 floats = 32 KiB).
#define LB_COLUMN_SUMS_NOALLOC_MAX_COLS 4096

// Per-column sum and sum of squares of a row-major [rows][cols] matrix of 16-bit floats:
//   out[c] = sum_r x[r][c],  out[cols + c] = sum_r x[r][c]^2      (fp32, OVERWRITTEN)
// Same numbers as lb_bn_partial_sums(x, sums, rows, cols, 1, dtype, 1, stream) writes into a
// zero-filled `sums`, but with no workspace argument and no allocation of any kind: the
// partial sums accumulate in a file-scope __device__ array of
// 2 * LB_COLUMN_SUMS_NOALLOC_MAX_COLS floats, which every call first clears on `stream`
// and finally copies to `out`.
//
//   dtype: 0 = fp16, 1 = bf16.  cols must be a multiple of 8 and x 16-byte aligned.
//
// Returns 0 on success; -1 for a null pointer, an x that is not 16-byte aligned, rows < 0,
// cols <= 0 or cols % 8 != 0, a dtype other than the two above, or a device index of 64 or
// more; -2 when cols exceeds LB_COLUMN_SUMS_NOALLOC_MAX_COLS (a message naming the limit
// goes to stderr); a positive cudaError_t if the set-up or a launch failed.
//
// Set-up: the FIRST call on each device looks the workspace's address up with
// cudaGetSymbolAddress (checked), which may load the module; make that call once outside
// any stream capture.  Later calls only enqueue work on `stream`.
//
// Concurrency: all calls on one device share the one workspace.  Calls that may overlap
// in time (different streams, or different host threads) race on it and give wrong sums;
// serialise them on one stream.
int lb_column_sums_noalloc(const void* x, float* out, long long rows, int cols, int dtype,
                           void* stream);

#ifdef __cplusplus
}
#endif
