// Layout of a rank's peer-writable inbox and of the communicator handle, shared by the kernels that
// talk to peers (the all-reduce, the pushing projections, the gathering norm, the LM-head exchange).
//
//   data  [2][world][max_bytes]      double buffered, one slot per source rank     (one-shot all-reduce)
//   flags [2][world][kMaxCtas]       epoch-valued arrival flags
//   Control                          device-resident bookkeeping (epochs, tickets, status)
//   line regions 0..kLlRegions-1     [2][world][kLlSlotBytes] each: 16-byte lines {data, epoch, data, epoch}
#pragma once

#include <stddef.h>
#include <stdint.h>

#include "common.cuh"

struct lri_comm {
  int rank, world;
  int64_t max_bytes;   // per slot
  uint8_t* local;      // this rank's inbox (cudaMalloc)
  uint8_t* peer[8];    // every rank's inbox as seen from this rank (peer[rank] == local)
  size_t total_bytes;
};

namespace lri {

constexpr int kMaxWorld = 8;
constexpr int kMaxCtas = 64;
constexpr int kArThreads = 256;

struct Control {
  unsigned int epoch;   // number of completed calls
  unsigned int ticket;  // CTAs retired in the running call
  int status;           // LRI_OK or LRI_ERR_TIMEOUT
  int pad;
  unsigned int chan_epoch[4];   // per line region 1..3: number of messages consumed by this rank
  unsigned int chan_ticket[4];  // per line region: consumer CTAs that have finished reading
};
static_assert(sizeof(Control) <= 64, "the control block has 64 bytes in the inbox");

__host__ __device__ inline size_t data_bytes(int world, int64_t max_bytes) {
  return static_cast<size_t>(2) * world * static_cast<size_t>(max_bytes);
}
__host__ __device__ inline size_t flags_offset(int world, int64_t max_bytes) { return data_bytes(world, max_bytes); }
__host__ __device__ inline size_t control_offset(int world, int64_t max_bytes) {
  return flags_offset(world, max_bytes) + static_cast<size_t>(2) * world * kMaxCtas * sizeof(unsigned int);
}

// Low-latency region: messages up to kLlMaxPayload bytes travel as 16-byte lines
// {data, epoch, data, epoch}: every 8-byte half carries its own arrival flag, so the receiver
// polls the data itself and neither a fence nor a separate flag store is on the critical path.
constexpr int64_t kLlMaxPayload = 128 * 1024;
constexpr int64_t kLlSlotBytes = 2 * kLlMaxPayload;
__host__ __device__ inline size_t ll_offset(int world, int64_t max_bytes) {
  return (control_offset(world, max_bytes) + 64 + 255) / 256 * 256;
}
__host__ __device__ inline size_t ll_bytes(int world) { return static_cast<size_t>(2) * world * kLlSlotBytes; }
// Line regions: region 0 belongs to lri_allreduce, regions 1..kPushChannels to the push channels
// (producer lri_comm_push / lri_linear_push, consumer lri_add_rmsnorm_gather), region kHeadRegion to
// the (value, index) exchange of the vocabulary-parallel LM head; each has its own epoch counter.
constexpr int kPushChannels = 2;
constexpr int kHeadRegion = 3;
constexpr int kLlRegions = 4;
__host__ __device__ inline size_t ll_region(int world, int64_t max_bytes, int region) {
  return ll_offset(world, max_bytes) + static_cast<size_t>(region) * ll_bytes(world);
}

}  // namespace lri
