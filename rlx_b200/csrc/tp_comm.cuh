// Layout of a rank's exchange buffer for the tensor-parallel sum (tp_comm.cu), shared with the down projection
// that pushes its tiles into it directly (gemv_int.cu).
//
// [header 1 KiB of 8-byte words] [parity 0: one slot of max_elems floats per possible rank] [parity 1: the same]
//   words 0..7    step counters of the stand-alone all-reduce, one per part (CTA)
//   words 8..71   its flags, [part][sending rank]
//   word  80      step counter of the fused form (advanced by the kernel in front of the pushing kernel)
//   word  81      CTA arrivals every rank will have counted in when that step is complete (cumulative)
//   word  82      CTAs of this rank's pushing kernels that have counted in (cumulative)
//   words 88..95  CTA arrivals of rank 0..7, added a whole grid at a time by that rank's last CTA to count in
#pragma once

#include <stdint.h>

namespace rlxq {

constexpr uint32_t kCommMaxWorld = 8;
constexpr uint32_t kCommParts = 8;            // CTAs per stand-alone all-reduce, each with its own counter and flags
constexpr uint32_t kCommHeader = 1024;
constexpr uint32_t kCommWordEpoch = 80, kCommWordExpected = 81, kCommWordLocal = 82, kCommWordArrive = 88;

// What a pushing kernel needs: every rank's buffer as mapped here, and who we are.
struct TpPush {
    uint8_t* buf[kCommMaxWorld];
    uint32_t world, rank, max_elems, spin_limit;
};

}  // namespace rlxq
