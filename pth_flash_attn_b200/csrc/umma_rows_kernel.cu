// Row-major tcgen05 attention kernel, head size 128 (query rows on the MMA M dimension).
#include <cuda.h>

#include "params.cuh"
#include "umma_rows.cuh"

namespace pthb200 {

__device__ unsigned int g_rows_status = 0;

// Reads and clears this file's status word (device must be idle).
cudaError_t read_rows_status(unsigned int* v) {
  unsigned int zero = 0;
  cudaError_t err = cudaMemcpyFromSymbol(v, g_rows_status, sizeof(*v));
  if (err != cudaSuccess) return err;
  return cudaMemcpyToSymbol(g_rows_status, &zero, sizeof(zero));
}

}  // namespace pthb200

#include "umma_rows_tile_test.cuh"
