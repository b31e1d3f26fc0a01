// Where a sharded decode call also writes its output rows: the same place of the gather window of every
// other rank (peer memory over NVLink), plus the flags that tell the ranks when a call's rows have all landed.
#pragma once

#include <stdint.h>

namespace mlxq {

constexpr int MAX_PEERS = 7;   // ranks beside this one (8 GPUs of one box)

struct PeerGather {
    int n;                          // peers written beside the local y (0: plain call)
    int rank;                       // this rank: the slot it owns in every rank's flag array
    unsigned epoch;                 // number of this gather call on the communicator (same on every rank)
    unsigned wait_epoch;            // before reading x, wait until every peer has finished this earlier call (0: none)
    char* y[MAX_PEERS];             // the local y pointer's twin inside each peer's window
    unsigned* flag[MAX_PEERS];      // each peer's flag array
    int peer_rank[MAX_PEERS];
    unsigned* my_flags;             // this rank's flag array: slot r holds the last epoch rank r finished
    unsigned* counter;              // CTAs of the running call that have stored all their rows (wraps at the grid size)
};

}  // namespace mlxq
