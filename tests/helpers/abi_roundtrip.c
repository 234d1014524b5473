/* A caller written in plain C, the way a non-Python host would use the library: only include/flame_offload.h,
 * the CUDA runtime for device memory, and (test infrastructure) the CPU oracle to check the bytes.
 * Mirrors round_trip_bf16 / pool-full / stale-handle of the reference's own tests
 * (src/activation_offload.rs:843-978) and adds the int8 block mode.
 *
 *   gcc -std=c99 abi_roundtrip.c -I include -I $CUDA/include -L flame_b200 -lflame_offload -L oracle -loracle \
 *       -L $CUDA/lib64 -lcudart -lm -o abi_roundtrip
 * Exit code 0 = every check passed. */
#define _POSIX_C_SOURCE 199309L
#include <cuda_runtime_api.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "flame_offload.h"

void oracle_quant_int8_b128(const uint16_t* in, int8_t* codes, float* scales, size_t n, unsigned flags);
void oracle_dequant_int8_b128(const int8_t* codes, const float* scales, uint16_t* out, size_t n);
uint16_t oracle_f32_to_bf16(float f);

#define CHECK(cond)                                                                                   \
  do {                                                                                                \
    if (!(cond)) {                                                                                    \
      fprintf(stderr, "FAILED %s:%d: %s  [%s]\n", __FILE__, __LINE__, #cond, flame_offload_last_error()); \
      return 1;                                                                                       \
    }                                                                                                 \
  } while (0)

static int wait_stream(cudaStream_t s) {  /* bounded: 20 s */
  int i;
  for (i = 0; i < 2000000; ++i) {
    cudaError_t e = cudaStreamQuery(s);
    if (e == cudaSuccess) return 0;
    if (e != cudaErrorNotReady) return 1;
    struct timespec ts = {0, 10000};
    nanosleep(&ts, NULL);
  }
  return 1;
}

int main(void) {
  const size_t n = 100000 + 37; /* not a multiple of 128, several 64 KiB chunks */
  size_t i;
  cudaStream_t st;
  CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) == cudaSuccess);
  uint16_t* h_in = (uint16_t*)flame_cuda_alloc_pinned_host(2 * n, 0);
  uint16_t* h_out = (uint16_t*)flame_cuda_alloc_pinned_host(2 * n, 0);
  CHECK(h_in && h_out);
  uint32_t lcg = 12345u;
  for (i = 0; i < n; ++i) {
    lcg = lcg * 1664525u + 1013904223u;
    float v = ((float)(lcg >> 8) / 8388608.0f - 1.0f) * ((i % 997 == 0) ? 40.0f : 1.5f);
    h_in[i] = oracle_f32_to_bf16(v);
  }
  void *d_in = NULL, *d_out = NULL;
  CHECK(cudaMalloc(&d_in, 2 * n) == cudaSuccess && cudaMalloc(&d_out, 2 * n) == cudaSuccess);
  CHECK(flame_h2d_async(d_in, h_in, 2 * n, st) == FLAME_OFFLOAD_OK);

  /* uncompressed: bit-exact round trip, accessors, pool full, stale handle */
  FlameOffloadPool* pool = flame_offload_pool_create(2, 2 * n, FLAME_OFFLOAD_COMPRESSION_NONE, NULL);
  CHECK(pool != NULL);
  CHECK(flame_offload_pool_num_slots(pool) == 2 && flame_offload_pool_slot_bytes(pool) == 2 * n);
  CHECK(flame_offload_pool_host_bytes(pool) == 2 * 2 * n && flame_offload_pool_in_flight(pool) == 0);
  FlameOffloadHandle h0, h1, h2;
  CHECK(flame_offload_pool_push(pool, d_in, n, FLAME_OFFLOAD_DTYPE_BF16, st, &h0) == FLAME_OFFLOAD_OK);
  CHECK(flame_offload_pool_push(pool, d_in, n, FLAME_OFFLOAD_DTYPE_BF16, st, &h1) == FLAME_OFFLOAD_OK);
  CHECK(flame_offload_pool_push(pool, d_in, n, FLAME_OFFLOAD_DTYPE_BF16, st, &h2) == FLAME_OFFLOAD_ERR_STATE);
  CHECK(strstr(flame_offload_last_error(), "ActivationOffloadPool full") != NULL);
  CHECK(flame_offload_pool_in_flight(pool) == 2);
  CHECK(flame_offload_pool_pull_into(pool, h1, d_out, 2 * n, st, 0) == FLAME_OFFLOAD_OK);
  CHECK(flame_d2h_async(h_out, d_out, 2 * n, st) == FLAME_OFFLOAD_OK);
  CHECK(wait_stream(st) == 0);
  CHECK(memcmp(h_in, h_out, 2 * n) == 0);
  CHECK(flame_offload_pool_pull_into(pool, h1, d_out, 2 * n, st, 0) == FLAME_OFFLOAD_ERR_STATE); /* double pull */
  CHECK(flame_offload_pool_clear(pool) == FLAME_OFFLOAD_OK);
  CHECK(flame_offload_pool_pull_into(pool, h0, d_out, 2 * n, st, 0) == FLAME_OFFLOAD_ERR_STATE); /* stale epoch */
  CHECK(strstr(flame_offload_last_error(), "stale") != NULL);
  CHECK(flame_offload_pool_synchronize(pool, 20.0) == FLAME_OFFLOAD_OK);
  flame_offload_pool_destroy(pool);

  /* int8 per 128: what the pinned slab holds and what comes back, against the oracle */
  FlameOffloadPoolConfig cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.struct_size = sizeof(cfg);
  cfg.device = -1;
  cfg.numa_node = -1;
  cfg.chunk_bytes = 64u << 10;
  pool = flame_offload_pool_create(1, 2 * n, FLAME_OFFLOAD_COMPRESSION_INT8_B128, &cfg);
  CHECK(pool != NULL);
  CHECK(flame_offload_pool_push(pool, d_in, n, FLAME_OFFLOAD_DTYPE_BF16, st, &h0) == FLAME_OFFLOAD_OK);
  const size_t nb = (n + 127) / 128;
  int8_t* codes = (int8_t*)malloc(n);
  int8_t* want_codes = (int8_t*)malloc(n);
  float* scales = (float*)malloc(4 * nb);
  float* want_scales = (float*)malloc(4 * nb);
  uint16_t* want_out = (uint16_t*)malloc(2 * n);
  CHECK(codes && want_codes && scales && want_scales && want_out);
  CHECK(flame_offload_pool_read_slot(pool, h0, codes, scales, 20.0) == FLAME_OFFLOAD_OK);
  oracle_quant_int8_b128(h_in, want_codes, want_scales, n, 0);
  CHECK(memcmp(codes, want_codes, n) == 0);
  CHECK(memcmp(scales, want_scales, 4 * nb) == 0);
  CHECK(flame_offload_pool_pull_into(pool, h0, d_out, 2 * n, st, 0) == FLAME_OFFLOAD_OK);
  CHECK(flame_d2h_async(h_out, d_out, 2 * n, st) == FLAME_OFFLOAD_OK);
  CHECK(wait_stream(st) == 0);
  oracle_dequant_int8_b128(want_codes, want_scales, want_out, n);
  CHECK(memcmp(h_out, want_out, 2 * n) == 0);
  FlameOffloadStats stats;
  CHECK(flame_offload_pool_stats(pool, &stats) == FLAME_OFFLOAD_OK);
  CHECK(stats.pushes == 1 && stats.pulls == 1 && stats.bytes_logical_out == 2 * n && stats.bytes_link_out < 2 * n * 53 / 100);
  flame_offload_pool_destroy(pool);

  free(codes); free(want_codes); free(scales); free(want_scales); free(want_out);
  cudaFree(d_in); cudaFree(d_out);
  CHECK(flame_cuda_free_pinned_host(h_in) == 0 && flame_cuda_free_pinned_host(h_out) == 0);
  cudaStreamDestroy(st);
  printf("abi_roundtrip: ok\n");
  return 0;
}
