// C ABI of the reference-GPU checker library (test infrastructure only).
//
// Each ref_gpu_* function wraps one GPU driver emitted by the reference's compiler
// (<kernel>_gpu_i32_f32; emitter src/backend/stitch_and_generate_gpu.cpp:141-161), compiled
// unchanged for sm_100a. All pointers are device pointers; the drivers run on stream 0 with
// the grid the caller names (the reference's default is 256 x 256,
// src/backend/generate_bindings.cpp:317-327). Result arrays are separate cudaMallocAsync
// allocations made by the emitted driver; release each with ref_gpu_free(). Every call
// synchronises the device before it returns and returns the CUDA error code seen (0 = none).
//
// The emitted SpGEMM keeps its product counters in int32 (src/backend/compute.cpp:541-611):
// callers must keep the product count of a call below 2^31.
#pragma once
#include <stddef.h>

#include "ref_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

int ref_gpu_free(void *p);
int ref_gpu_copy(void *dst, const void *src, size_t bytes);  // device to device, synchronous
int ref_gpu_csr_add(const ref_csr *a, const ref_csr *b, ref_csr *z, int num_blocks, int threads_per_block);
int ref_gpu_csr_mul(const ref_csr *a, const ref_csr *b, ref_csr *z, int num_blocks, int threads_per_block);
int ref_gpu_csr_add_3(const ref_csr *a, const ref_csr *b, const ref_csr *c, ref_csr *z, int num_blocks, int threads_per_block);
int ref_gpu_spgemm(const ref_csr *a, const ref_csr *b, ref_csr *z, int num_blocks, int threads_per_block);
int ref_gpu_sssmm(const ref_csr *a, const ref_csr *b, const ref_csr *c, ref_csr *z, int num_blocks, int threads_per_block);
int ref_gpu_coo3d_add(const ref_coo3 *a, const ref_coo3 *b, ref_coo3 *z, int num_blocks, int threads_per_block);
int ref_gpu_csf_add(const ref_csf3 *a, const ref_csf3 *b, ref_csf3 *z, int num_blocks, int threads_per_block);

#ifdef __cplusplus
}
#endif
