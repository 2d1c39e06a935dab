// Shared device-side definitions for the sm_100a kernel templates.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "genn_b200.h"
#include "genn_b200_rng.h"

namespace b200
{
// Step counters kept on the device so a captured step graph can be replayed
// without touching kernel arguments: `timestep` gives t = timestep * dt,
// `steps_done` drives every ring pointer (spike queue slot, dendritic-delay
// front), `ticket` elects the last block of the neuron kernel, `error` is set
// by bounds checks.
struct StepState
{
    unsigned long long timestep;
    unsigned long long steps_done;
    unsigned int ticket;
    unsigned int error;
    // steps_done modulo ring_period, a common multiple of every ring size (spike
    // queue depths, dendritic-delay depths), so ring slots come from 32-bit
    // arithmetic: (phase + c) % n == (steps_done + c) % n for every ring size n
    unsigned int phase;
    unsigned int ring_period;
    unsigned long long synaptic_events;   // only advanced when event counting is on
    unsigned long long spikes;
    // SM clock cycles CTA 0 spent in each phase of the persistent kernel:
    // presynaptic work, barrier after it, neuron work, barrier after it
    unsigned long long phase_cycles[4];
    unsigned long long probe[12];        // finer clock64 sums of the persistent kernel's profile mode
    // verdict of tiledDecideKernel for the step being delivered: 1 = enough events for the
    // target-tiled kernel, 0 = the one-reduction-per-event kernel delivers
    unsigned int heavy;
    // most spikes (all populations and batch entries together) any step has emitted since the host last
    // read and cleared this word: tells the host whether launching the tiled kernels is worth it at all
    unsigned int peak_spikes;
    // limits of every wait inside the persistent kernels (set by the host; a wait that runs out sets an
    // error bit, all CTAs leave the kernel and the host reports it): polls of the grid barrier, polls for
    // a word another process writes, SM cycles a warp waits for work from another warp of its CTA
    unsigned long long barrier_spin_limit;
    unsigned long long exchange_spin_limit;
    long long stream_wait_cycles;
};

constexpr unsigned int ERR_SPIKE_OVERFLOW = 1u;
constexpr unsigned int ERR_IND_RANGE = 2u;
constexpr unsigned int ERR_DELAY_RANGE = 4u;

// Block -> merged-group element lookup: block_start[g] is the first block of
// group g, block_start[num_groups] the grid size.  Linear for a handful of
// groups, binary beyond that (the reference emits the same two forms,
// backendSIMT.h:244-323).
__device__ __forceinline__ unsigned int findGroup(const unsigned int *__restrict__ block_start,
                                                  unsigned int num_groups, unsigned int block)
{
    // plain loads: the table may live in shared memory
    if(num_groups <= 8) {
        unsigned int g = 0;
        while(g + 1 < num_groups && block >= block_start[g + 1]) g++;
        return g;
    }
    unsigned int lo = 0, hi = num_groups;
    while(hi - lo > 1) {
        const unsigned int mid = (lo + hi) >> 1;
        if(block >= block_start[mid]) lo = mid; else hi = mid;
    }
    return lo;
}

// fp32 add to GLOBAL memory with no return value.  The address space is spelled out: after a
// reduction through a generic pointer the load/store unit holds back later generic accesses
// (the staged tables in shared memory are read through generic pointers) until it completes.
__device__ __forceinline__ void redAdd(float *addr, float v)
{
    asm volatile("red.global.add.f32 [%0], %1;" :: "l"(__cvta_generic_to_global(addr)), "f"(v));
}

__device__ __forceinline__ unsigned int ringSlot(unsigned int k, unsigned int slots)
{
    return k % slots;
}
}   // namespace b200
