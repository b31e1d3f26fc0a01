// Where a sharded decode call also writes its output rows: the same place of the gather window of every
// other rank (peer memory over NVLink), plus the flags that tell the ranks when a call's rows have all landed.
#pragma once

#include <stdint.h>

namespace mlxq {

constexpr int MAX_PEERS = 7;   // ranks beside this one (8 GPUs of one box)

struct PeerGather {
    int n;                          // peers written beside the local y (0: plain call)
    int rank;                       // this rank: the slot it owns in every rank's flag array
    unsigned epoch;                 // number of this gather call on the communicator (same on every rank); before it reads x the
                                    // kernel waits until every peer has finished call epoch - 1 (whose rows may be this call's x)
    char* y[MAX_PEERS];             // the local y pointer's twin inside each peer's window
    unsigned* flag[MAX_PEERS];      // each peer's flag array
    int peer_rank[MAX_PEERS];
    unsigned* my_flags;             // this rank's flag array: word r is the number of rank r's calls whose rows are complete
                                    // everywhere (published by the kernel that follows a call, so also: rank r has started call word + 1)
    unsigned* counter;              // CTAs of the running call that have published their rows (wraps at the grid size)
    int x_is_gathered;              // the activations lie in this rank's gather window (a previous call's output): wait for
                                    // the peers before reading them; otherwise the wait is put off until the first row is stored
    unsigned* epoch_ctr;            // device word holding the number of completed gather calls; when set, the kernel takes
                                    // its epoch from it (completed + 1) instead of `epoch`, so that a captured launch can be replayed
};

}  // namespace mlxq
