// Layout of a rank's exchange buffer for the tensor-parallel sum (tp_comm.cu), shared with the down projection
// that pushes its tiles into it directly (gemv_int.cu).
//
// [header 1 KiB of 8-byte words] [parity 0: one slot of max_elems tagged 8-byte words {value, step tag} per possible
// rank] [parity 1: the same] [the pushing down projection's float slots: parity 0, parity 1, max_elems floats per rank]
//   words 0..7    step counters of the stand-alone all-reduce, one per part (CTA)
//   word  80      step counter of the fused form (advanced by the kernel in front of the pushing kernel)
//   word  81      CTA arrivals every rank will have counted in when that step is complete (cumulative)
//   word  82      CTAs of this rank's pushing kernels that have counted in (cumulative)
//   words 88..95  CTA arrivals of rank 0..7, added a whole grid at a time by that rank's last CTA to count in
#pragma once

#include <stdint.h>

namespace rlxq {

constexpr uint32_t kCommMaxWorld = 8;
constexpr uint32_t kCommParts = 8;            // CTAs per stand-alone all-reduce, each with its own step counter
constexpr uint32_t kCommHeader = 1024;
constexpr uint32_t kCommWordEpoch = 80, kCommWordExpected = 81, kCommWordLocal = 82, kCommWordArrive = 88;

// byte offset of the pushing down projection's float slots in a buffer
__host__ __device__ inline size_t comm_push_offset(uint32_t max_elems) {
    return kCommHeader + 2 * (size_t)kCommMaxWorld * max_elems * 8;
}

// What a pushing kernel needs: every rank's buffer as mapped here, and who we are.
struct TpPush {
    uint8_t* buf[kCommMaxWorld];
    uint32_t world, rank, max_elems, spin_limit;
};

}  // namespace rlxq
