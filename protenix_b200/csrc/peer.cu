// Buffers that the other GPUs of the box can write into, and the strided copy that fills them.
//
// The row-sharded path exchanges slabs between GPUs (row shards <-> channel shards, row shards <-> column shards).
// Every one of those exchanges is a set of pitched 2-D copies from a local tensor straight into its final place in a
// peer's receive buffer, so no re-layout pass is needed on either side.  The buffers are plain cudaMalloc
// allocations exported through CUDA IPC; the copy is a hand-written kernel with 16-byte loads from local memory and
// 16-byte stores to peer memory over NVLink (no TMA, no multicast).  No counterpart in the reference.
//
// Ordering between the GPUs is a barrier of flags in peer memory (px_peer_barrier): every rank stores the number of
// the barrier into its slot of every other rank's flag array (a system-scope release, after its earlier copies in
// the stream) and then waits, with a limit, until its own array shows that number from every rank (system-scope
// acquires).  One small kernel per rank instead of a collective; a rank that never arrives makes the others give
// up after the wait limit and leaves a flag for the host, the context stays usable.
#include <cstring>

#include "px_tcgen05.cuh"

namespace px {

struct BarrierPeers {
  unsigned int* flags[PX_COPY_BATCH_MAX];   // flags[r]: the flag array of rank r, as mapped into this process
};

// One warp.  Lane r < world stores `epoch` into slot `rank` of rank r's array, then waits for slot r of its own.
// Barrier numbers only grow, so "reached" is a signed comparison of the difference and nothing is ever reset.
__global__ void __launch_bounds__(32) peer_barrier_kernel(BarrierPeers peers, int rank, int world, unsigned int epoch) {
  const int r = threadIdx.x;
  if (r < world && r != rank) {
    asm volatile("fence.acq_rel.sys;\n" ::: "memory");
    asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(peers.flags[r] + rank), "r"(epoch) : "memory");
    const unsigned int* mine = peers.flags[rank] + r;
    const long long t0 = clock64();
    const long long limit = *reinterpret_cast<volatile long long*>(&g_wait_limit);
    for (;;) {
      unsigned int seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(mine) : "memory");
      if ((int)(seen - epoch) >= 0) break;
      if (clock64() - t0 > limit) {               // rank r never arrived
        atomicOr(&g_tc_error, 1u << (r & 15));
        break;
      }
      __nanosleep(64);
    }
  }
}

// Rows of `units` 16-byte pieces; one thread per piece, grid-stride over rows x pieces.  128 threads and few
// registers per CTA, so that a copy can take the room the persistent compute kernels leave on an SM (they hold up
// to 61440 of its 65536 registers) and run beside them on another stream.
__global__ void __launch_bounds__(128)
copy_2d_kernel(uint4* __restrict__ dst, long long dpitch16, const uint4* __restrict__ src, long long spitch16,
               long long units, long long height) {
  const long long total = units * height, step = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  // four pieces in flight per thread: the loads from local memory overlap, the stores to peer memory are posted
  for (; i + 3 * step < total; i += 4 * step) {
    uint4 v[4];
    long long at[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const long long j = i + k * step, r = j / units, c = j - r * units;
      v[k] = __ldcs(src + r * spitch16 + c);
      at[k] = r * dpitch16 + c;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) dst[at[k]] = v[k];
  }
  for (; i < total; i += step) {
    const long long r = i / units, c = i - r * units;
    dst[r * dpitch16 + c] = src[r * spitch16 + c];
  }
}

// The same copy to up to 16 destinations in one launch (blockIdx.y = destination): the exchanges of the row-sharded
// path send one block of identical shape to every rank.
struct CopyBatch {
  uint4* dst[PX_COPY_BATCH_MAX];
  const uint4* src[PX_COPY_BATCH_MAX];
};
__global__ void __launch_bounds__(128)
copy_2d_batch_kernel(CopyBatch b, long long dpitch16, long long spitch16, long long units, long long height) {
  uint4* __restrict__ dst = b.dst[blockIdx.y];
  const uint4* __restrict__ src = b.src[blockIdx.y];
  const long long total = units * height, step = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  // four pieces in flight per thread: the loads from local memory overlap, the stores to peer memory are posted
  for (; i + 3 * step < total; i += 4 * step) {
    uint4 v[4];
    long long at[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const long long j = i + k * step, r = j / units, c = j - r * units;
      v[k] = __ldcs(src + r * spitch16 + c);
      at[k] = r * dpitch16 + c;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) dst[at[k]] = v[k];
  }
  for (; i < total; i += step) {
    const long long r = i / units, c = i - r * units;
    dst[r * dpitch16 + c] = src[r * spitch16 + c];
  }
}

PX_DEFINE_FAMILY_HOOKS(peer)

}  // namespace px

using namespace px;

extern "C" int32_t px_peer_barrier(void* const* flag_arrays, int32_t rank, int32_t world, uint32_t epoch, void* stream) {
  if (!flag_arrays || world <= 0 || world > PX_COPY_BATCH_MAX || rank < 0 || rank >= world) return PX_ERR_BAD_ARG;
  BarrierPeers p;
  for (int i = 0; i < PX_COPY_BATCH_MAX; ++i) {
    p.flags[i] = (unsigned int*)flag_arrays[i < world ? i : rank];
    if (!p.flags[i] || ((uintptr_t)p.flags[i] & 3)) return PX_ERR_BAD_ARG;
  }
  if (world == 1) return PX_OK;
  peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(p, rank, world, epoch);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

static_assert(sizeof(cudaIpcMemHandle_t) == PX_PEER_HANDLE_BYTES, "handle size");

extern "C" int32_t px_peer_alloc(int64_t bytes, void** ptr, unsigned char* handle) {
  if (bytes <= 0 || !ptr || !handle) return PX_ERR_BAD_ARG;
  void* p = nullptr;
  if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) return PX_ERR_WORKSPACE;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    cudaFree(p);
    return PX_ERR_LAUNCH;
  }
  memcpy(handle, &h, sizeof(h));
  *ptr = p;
  return PX_OK;
}

extern "C" int32_t px_peer_open(const unsigned char* handle, void** ptr) {
  if (!handle || !ptr) return PX_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return PX_ERR_LAUNCH;
  *ptr = p;
  return PX_OK;
}

extern "C" int32_t px_peer_close(void* ptr) {
  if (!ptr) return PX_ERR_BAD_ARG;
  return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

extern "C" int32_t px_peer_free(void* ptr) {
  if (!ptr) return PX_ERR_BAD_ARG;
  return cudaFree(ptr) == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

extern "C" int32_t px_copy_2d(void* dst, int64_t dpitch, const void* src, int64_t spitch, int64_t width_bytes,
                              int64_t height, void* stream) {
  if (!dst || !src || width_bytes < 0 || height < 0 || dpitch < width_bytes || spitch < width_bytes) return PX_ERR_BAD_ARG;
  if (((uintptr_t)dst | (uintptr_t)src | (uintptr_t)dpitch | (uintptr_t)spitch | (uintptr_t)width_bytes) & 15)
    return PX_ERR_BAD_ARG;
  if (width_bytes == 0 || height == 0) return PX_OK;
  const long long units = width_bytes / 16, total = units * height;
  long long blocks = (total + 127) / 128;
  if (blocks > 148 * 16) blocks = 148 * 16;
  copy_2d_kernel<<<(unsigned)blocks, 128, 0, (cudaStream_t)stream>>>((uint4*)dst, dpitch / 16, (const uint4*)src, spitch / 16,
                                                                     units, height);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}

// The same copy by the GPU's copy engines (one pitched cudaMemcpy2DAsync): no SM is involved, so it overlaps any
// kernel.  Worth it for wide rows; narrow rows (a few hundred bytes) are better served by the kernel above.
extern "C" int32_t px_copy_2d_dma(void* dst, int64_t dpitch, const void* src, int64_t spitch, int64_t width_bytes,
                                  int64_t height, void* stream) {
  if (!dst || !src || width_bytes < 0 || height < 0 || dpitch < width_bytes || spitch < width_bytes) return PX_ERR_BAD_ARG;
  if (width_bytes == 0 || height == 0) return PX_OK;
  return cudaMemcpy2DAsync(dst, (size_t)dpitch, src, (size_t)spitch, (size_t)width_bytes, (size_t)height, cudaMemcpyDefault,
                           (cudaStream_t)stream) == cudaSuccess
             ? PX_OK
             : PX_ERR_LAUNCH;
}

extern "C" int32_t px_copy_2d_batch(void* const* dst, const void* const* src, int32_t count, int64_t dpitch, int64_t spitch,
                                    int64_t width_bytes, int64_t height, void* stream) {
  if (!dst || !src || count <= 0 || count > PX_COPY_BATCH_MAX || width_bytes < 0 || height < 0 || dpitch < width_bytes ||
      spitch < width_bytes)
    return PX_ERR_BAD_ARG;
  if (((uintptr_t)dpitch | (uintptr_t)spitch | (uintptr_t)width_bytes) & 15) return PX_ERR_BAD_ARG;
  CopyBatch b;
  for (int i = 0; i < PX_COPY_BATCH_MAX; ++i) {
    const int j = i < count ? i : 0;
    if (!dst[j] || !src[j] || (((uintptr_t)dst[j] | (uintptr_t)src[j]) & 15)) return PX_ERR_BAD_ARG;
    b.dst[i] = (uint4*)dst[j];
    b.src[i] = (const uint4*)src[j];
  }
  if (width_bytes == 0 || height == 0) return PX_OK;
  const long long units = width_bytes / 16, total = units * height;
  long long blocks = (total + 127) / 128;
  const long long cap = (148 * 16 + count - 1) / count;
  if (blocks > cap) blocks = cap;
  copy_2d_batch_kernel<<<dim3((unsigned)blocks, (unsigned)count), 128, 0, (cudaStream_t)stream>>>(b, dpitch / 16, spitch / 16, units,
                                                                                              height);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}
