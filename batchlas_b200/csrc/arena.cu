// Per-queue workspace arena backed by a stream-ordered memory pool of its own: every arena creates
// one cudaMemPool_t on its device (cudaMemPoolCreate) and takes its blocks from it with
// cudaMallocFromPoolAsync on the queue's stream, so a queue's scratch never mixes with the
// application's default pool, trim() really returns the bytes to the driver (cudaMemPoolTrimTo), and
// destroying the queue destroys the pool.
//
// Lease semantics follow BatchLAS's WorkspaceArena (src/queue.hh:41-226) and WorkspaceLease
// (include/util/workspace.hh:70-162):
//   * a borrow is carved from the current block at an aligned cursor; when nothing from the
//     current block onward fits, a new block of max(request, 2 * last block, 64 KiB) is opened,
//     so leased memory never moves and a ratcheting caller allocates O(log) times;
//   * releasing the innermost outstanding loan rewinds the cursor to where that loan started,
//     and then also reclaims any loans beneath it that were already returned out of order;
//   * releasing any other loan only marks it; its bytes stay reserved until it becomes innermost;
//   * trim() refuses while any loan is outstanding, otherwise drains the stream and frees all.
// The reference's blocks are shared USM; here they are device memory of the arena's own pool.
#include <algorithm>
#include <new>
#include <stdlib.h>
#include <vector>

#include "common.cuh"

struct blb200_arena {
  struct Block {
    char* ptr;
    size_t size;
  };
  struct LiveLoan {
    uint64_t seq;
    size_t block, offset;
    bool returned;
  };
  int device;  // < 0: host malloc backing (bookkeeping tests without a GPU)
  cudaStream_t stream;
  cudaMemPool_t pool = nullptr;  // created with the first block
  size_t align;
  std::vector<Block> blocks;
  size_t cur_block = 0, cur_offset = 0;
  std::vector<LiveLoan> live;
  uint64_t next_seq = 0;

  int alloc_block(size_t bytes, char** out) {
    if (device < 0) {
      void* p = nullptr;
      if (posix_memalign(&p, align, bytes) != 0) return BLB200_E_INTERNAL;
      *out = (char*)p;
      return BLB200_OK;
    }
    if (!pool) {
      cudaMemPoolProps props = {};
      props.allocType = cudaMemAllocationTypePinned;  // ordinary device memory
      props.handleTypes = cudaMemHandleTypeNone;
      props.location.type = cudaMemLocationTypeDevice;
      props.location.id = device;
      cudaError_t e = cudaMemPoolCreate(&pool, &props);
      if (e != cudaSuccess) return (int)e;
    }
    void* p = nullptr;
    cudaError_t e = cudaMallocFromPoolAsync(&p, bytes, pool, stream);
    if (e != cudaSuccess) return (int)e;
    *out = (char*)p;
    return BLB200_OK;
  }
  void free_all() {
    for (auto& b : blocks) {
      if (device < 0)
        free(b.ptr);
      else
        cudaFreeAsync(b.ptr, stream);
    }
    blocks.clear();
    cur_block = cur_offset = 0;
    live.clear();  // next_seq keeps counting: a sequence number is never handed out twice
  }
};

extern "C" {

int blb200_arena_create(int device, void* cuda_stream, blb200_arena** out) {
  if (!out) return BLB200_E_NULL;
  blb200_arena* a = new (std::nothrow) blb200_arena();
  if (!a) return BLB200_E_INTERNAL;
  a->device = device;
  a->stream = (cudaStream_t)cuda_stream;
  // The reference aligns to max(16, mem_base_addr_align / 8); CUDA devices report 4096 bits
  // there, i.e. 512 bytes, which is also what cudaMalloc* guarantees at least 256 of.
  a->align = 512;
  *out = a;
  return BLB200_OK;
}

int blb200_arena_destroy(blb200_arena* a) {
  if (!a) return BLB200_E_NULL;
  if (a->device >= 0 && !a->blocks.empty()) cudaStreamSynchronize(a->stream);
  a->free_all();
  if (a->pool) {
    cudaStreamSynchronize(a->stream);  // the frees above are stream-ordered
    cudaMemPoolDestroy(a->pool);
  }
  delete a;
  return BLB200_OK;
}

int blb200_arena_acquire(blb200_arena* a, size_t bytes, blb200_lease* out) {
  if (!a || !out) return BLB200_E_NULL;
  const size_t al = a->align;
  const size_t want = (bytes + al - 1) & ~(al - 1);
  auto record = [&](char* ptr, size_t block, size_t offset) {
    const uint64_t seq = ++a->next_seq;  // 0 stays "no loan"
    a->live.push_back({seq, block, offset, false});
    out->ptr = ptr;
    out->bytes = bytes;
    out->block = block;
    out->offset = offset;
    out->seq = seq;
  };
  // Blocks before cur_block are spoken for by outstanding leases.
  while (a->cur_block < a->blocks.size()) {
    const size_t off = (a->cur_offset + al - 1) & ~(al - 1);
    if (off + want <= a->blocks[a->cur_block].size) {
      a->cur_offset = off + want;
      record(a->blocks[a->cur_block].ptr + off, a->cur_block, off);
      return BLB200_OK;
    }
    ++a->cur_block;
    a->cur_offset = 0;
  }
  const size_t last = a->blocks.empty() ? 0 : a->blocks.back().size;
  const size_t block_size = std::max({want, last * 2, (size_t)64 * 1024});
  char* p = nullptr;
  int rc = a->alloc_block(block_size, &p);
  if (rc != BLB200_OK) {
    a->cur_block = a->blocks.empty() ? 0 : a->blocks.size() - 1;
    return rc;
  }
  a->blocks.push_back({p, block_size});
  a->cur_block = a->blocks.size() - 1;
  a->cur_offset = want;
  record(p, a->cur_block, 0);
  return BLB200_OK;
}

int blb200_arena_release(blb200_arena* a, const blb200_lease* lease) {
  if (!a || !lease) return BLB200_E_NULL;
  if (lease->seq == 0) return BLB200_OK;  // empty or already released handle
  if (!a->live.empty() && a->live.back().seq == lease->seq) {
    a->live.pop_back();
    a->cur_block = lease->block;
    a->cur_offset = lease->offset;
    while (!a->live.empty() && a->live.back().returned) {
      a->cur_block = a->live.back().block;
      a->cur_offset = a->live.back().offset;
      a->live.pop_back();
    }
    return BLB200_OK;
  }
  for (auto it = a->live.rbegin(); it != a->live.rend(); ++it)
    if (it->seq == lease->seq) {
      it->returned = true;
      return BLB200_OK;
    }
  return BLB200_OK;  // unknown sequence number: stale handle after a trim; nothing to do
}

int blb200_arena_trim(blb200_arena* a) {
  if (!a) return BLB200_E_NULL;
  if (!a->live.empty()) return 0;
  if (a->blocks.empty()) return 1;
  if (a->device >= 0) {
    cudaError_t e = cudaStreamSynchronize(a->stream);
    if (e != cudaSuccess) return BLB200_E_INTERNAL;
  }
  a->free_all();
  if (a->pool) {
    cudaStreamSynchronize(a->stream);  // the frees above are stream-ordered
    cudaMemPoolTrimTo(a->pool, 0);     // back to the driver, as the reference's trim frees its USM blocks
  }
  return 1;
}

size_t blb200_arena_capacity(const blb200_arena* a) {
  size_t total = 0;
  if (a)
    for (auto& b : a->blocks) total += b.size;
  return total;
}

size_t blb200_arena_block_count(const blb200_arena* a) { return a ? a->blocks.size() : 0; }
size_t blb200_arena_alignment(const blb200_arena* a) { return a ? a->align : 0; }

}  // extern "C"
