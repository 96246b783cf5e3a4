// Chunk tables of the attention kernels (context parallelism without gathered K/V).
//
// Logical key position x -> (source buffer, row inside it), and local query row -> absolute
// position.  With all fields zero the tables describe the plain case: one K/V buffer in logical
// order and queries that start at the kernel's q_offset.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace kb {

constexpr int MAX_KV_SRC = 8;       // K/V source buffers (context-parallel ranks)
constexpr int MAX_KV_CHUNKS = 16;   // logical chunks (two per rank)
constexpr int MAX_Q_CHUNKS = 2;     // local query chunks (dual-chunk ownership)

struct KvMaps {
  CUtensorMap k[MAX_KV_SRC];
  CUtensorMap v[MAX_KV_SRC];
};

struct ChunkGeom {
  int kv_chunk_rows;                 // 0: single source in logical order
  int kv_src[MAX_KV_CHUNKS];
  int kv_row_base[MAX_KV_CHUNKS];
  int q_chunk_rows;                  // 0: one query chunk starting at the kernel's q_offset
  int q_pos[MAX_Q_CHUNKS];

  // source buffer and row of logical key position x (x is a multiple of the 128-key tile and chunks
  // are multiples of 128 rows, so a tile never straddles two chunks)
  __host__ __device__ inline void locate(int x, int& src, int& row) const {
    if (kv_chunk_rows == 0) {
      src = 0;
      row = x;
      return;
    }
    const int c = x / kv_chunk_rows;
    src = kv_src[c];
    row = kv_row_base[c] + (x - c * kv_chunk_rows);
  }
  // offset o such that local query row x (in the 128-row tile starting at q0) has absolute position o + x
  __host__ __device__ inline int q_offset_of(int q0, int plain_offset) const {
    if (q_chunk_rows == 0) return plain_offset;
    const int c = q0 / q_chunk_rows;
    return q_pos[c] - c * q_chunk_rows;
  }
};

// Validates and fills a ChunkGeom from host arrays; returns 0 or 7 (bad argument).
inline int fill_chunk_geom(ChunkGeom* geom, int n_src, const int* kv_src, const int* kv_row_base, int n_chunks,
                           int chunk_rows, int src_rows, int q_chunk_rows, const int* q_pos, int sq) {
  *geom = ChunkGeom{};
  if (n_src < 1 || n_src > MAX_KV_SRC || n_chunks < 1 || n_chunks > MAX_KV_CHUNKS) return 7;
  if (chunk_rows <= 0 || chunk_rows % 128 || q_chunk_rows <= 0 || q_chunk_rows % 128 || sq % q_chunk_rows) return 7;
  if (sq / q_chunk_rows > MAX_Q_CHUNKS) return 7;
  geom->kv_chunk_rows = chunk_rows;
  for (int c = 0; c < n_chunks; ++c) {
    if (kv_src[c] < 0 || kv_src[c] >= n_src || kv_row_base[c] < 0 || kv_row_base[c] + chunk_rows > src_rows) return 7;
    geom->kv_src[c] = kv_src[c];
    geom->kv_row_base[c] = kv_row_base[c];
  }
  geom->q_chunk_rows = q_chunk_rows;
  for (int i = 0; i < sq / q_chunk_rows; ++i) geom->q_pos[i] = q_pos[i];
  return 0;
}

}  // namespace kb
