// What a CTA that gives up still has in flight.
//
// Every wait in this library's kernels is bounded. A wait that runs out means a fault in a kernel's protocol; the CTA
// records a code and leaves. The rule it keeps on the way out: it does not free tensor memory, and does not return (which
// hands its shared memory to the next CTA on the SM), while bulk copies it asked for can still land or tensor-core
// instructions it issued can still run. So, after setting the code, it waits -- bounded again -- for every "full"
// barrier that has been armed (expect_tx) and not yet waited for, and for a commit behind the last MMA it issued; only
// then come tcgen05.dealloc and the return. This header holds the bookkeeping of the first half, which is plain
// arithmetic and is tested on the host.
#pragma once

#include <cuda_runtime.h>

namespace sm {

// A ring of `stages` buffers is filled in order: fill f (counted from 0) goes into stage f % stages and completes the phase
// of parity (f / stages) & 1 of that stage's barrier. `issued` fills have been asked for (their barriers armed), the
// first `consumed` of them have been waited for. The others are outstanding: at most `stages` of them, since a stage is
// armed again only after it has been waited for.
struct OutstandingFill {
    int stage;
    unsigned parity;
};
__host__ __device__ inline int outstanding_fills(long long issued, long long consumed, int stages, OutstandingFill* out) {
    int n = 0;
    if (stages <= 0 || consumed < 0) return 0;
    for (long long f = consumed; f < issued && n < stages; ++f) {
        out[n].stage = (int)(f % stages);
        out[n].parity = (unsigned)((f / stages) & 1);
        ++n;
    }
    return n;
}

}  // namespace sm
