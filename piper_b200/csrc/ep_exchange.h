// Host-side launchers of the expert-parallel exchange kernels (ep_exchange.cu).
// Flag blocks are arrays of uint64 in symmetric memory; `*_off` arguments are
// word offsets of a block of `ep` words inside a rank's flag array.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace piper {

struct EpDispatchArgs {
  const void* x;                 // [T, D] bf16 tokens of this rank
  const int* idx;                // [T, k] expert of every (token, choice)
  const int* counts;             // [E] rows this rank routes to every expert
  const int* g_start_loc;        // [E] first row of expert e in this rank's own padded layout
  int* seg_off;                  // [E] scratch
  int* ctl;                      // [1 + ep] scratch
  int* cursor;                   // [E] zeros
  int* pos_loc;                  // [T * k] out: row of every copy in this rank's own padded layout
  void* const* peer_recv;        // [ep] receive buffer of this slot on every rank
  int* const* peer_meta;         // [ep] meta block of this slot on every rank (2 * ep * El ints)
  uint64_t* const* peer_flags;   // [ep] flag array of every rank
  const uint64_t* free_flags;    // local FREE block of the slot's receive buffer (one word per owner)
  unsigned long long free_needed;
  int ready_off;                 // READY block of the slot's receive buffer
  unsigned long long use;
  unsigned int* cta_counter;
  int my_rank, ep, experts_local;
  long long T;
  int D, k, cap_src;
  unsigned long long timeout_ns;
  int* status;
  int num_ctas;
};

// Gathers every (token, choice) row of x into the region that the owner of its expert keeps for this source
// rank, publishes the per-expert counts and local segment starts, then READY.  Rows for an owner whose region
// they would overflow are not sent (status = bad argument).
int ep_dispatch_push(const EpDispatchArgs& a, cudaStream_t st);

// Owner side: wait for all sources, then build the group table of the regions and the flat count vector
// [ep * experts_local] (source-major).
int ep_wait_table(const uint64_t* ready_flags, const int* meta, int* g_start, int* g_len, int* counts_out, int ep,
                  int experts_local, int cap_src, unsigned long long use, unsigned long long timeout_ns, int* status,
                  cudaStream_t st);

struct EpBlockPushArgs {
  const void* src;               // [src_rows, D] bf16
  const int* seg_src;            // [G] first source row of segment g
  const int* seg_len;            // [G] rows of segment g
  const int* seg_dst;            // [G] first destination row (before dst_bias)
  int num_segments, group_div, dst_bias;
  long long src_rows, dst_rows;
  void* const* peer_dst;         // [ep] destination buffer on every rank
  uint64_t* const* peer_flags;
  const uint64_t* free_flags;    // local FREE block of the destination buffers
  unsigned long long free_needed;
  int ready_off;
  unsigned long long use;
  unsigned int* cta_counter;
  int* abort;                    // one int of scratch: set by the FREE wait, read by the copy kernel
  int my_rank, ep, D;
  unsigned long long timeout_ns;
  int* status;
  int num_ctas;
};

// Copies row segments into peers' buffers (segment g to rank g / group_div) and publishes READY.
int ep_block_push(const EpBlockPushArgs& a, cudaStream_t st);

// One-thread kernels: wait until flags[0..n) >= value (`tag` is reported if the wait runs out;
// abort[0], if given, becomes 1 then and 0 otherwise); store value into word (off + my_rank) of every rank.
int ep_wait(const uint64_t* flags, int n, unsigned long long value, unsigned long long timeout_ns, int* status,
            int tag, int* abort, cudaStream_t st);
int ep_signal(uint64_t* const* peer_flags, int off, int my_rank, int ep, unsigned long long value, cudaStream_t st);

}  // namespace piper
