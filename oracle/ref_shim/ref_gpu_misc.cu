// Deallocation for the reference-GPU checker library: the emitted drivers allocate every result
// array with cudaMallocAsync on stream 0 (runtime/nacho_nb.h:50-58 frees them the same way).
#include "ref_gpu_common.h"

extern "C" int ref_gpu_free(void *p) {
    if (!p) return 0;
    return (int)cudaFreeAsync(p, 0);
}

extern "C" int ref_gpu_copy(void *dst, const void *src, size_t bytes) {
    if (!bytes) return 0;
    return (int)cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToDevice);
}
