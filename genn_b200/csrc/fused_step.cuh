// Persistent fused time-step kernel: many simulation steps in ONE cooperative
// launch, the presynaptic update and the neuron update separated by grid-wide
// barriers instead of kernel boundaries.
//
// The reference issues 2-7 tiny kernels per step on stream 0
// (backendCUDAHIP.cc:386-420, 548-589).  On the Potjans microcircuit a step
// moves under a megabyte, so its cost is launch and dependency latency, not
// bandwidth.  Here one CTA set stays resident (cooperative launch, a multiple of
// the SM count) and loops over the steps:
//
//   phase A  presynaptic update, work item = (spike, 128-synapse chunk of its
//            row), one WARP per item, items of all merged SPARSE groups
//            flattened: every warp reads the spike counts of all sources with
//            one lane each, prefix-sums them with shuffles and strides through
//            the item space.  Spike ids are fetched with the counts (one round
//            trip), the row length with the row data (one more).
//   barrier  (reductions into outPost/denDelay must have landed)
//   phase B  neuron update of every merged group, one thread per neuron, spike
//            emission with warp-aggregated atomics; one thread clears the spike
//            counts of the slot the next step writes.
//   barrier  (spike lists complete)
//
// Two barriers per step are inherent while zero-step dendritic delays exist
// (a synapse with d = 0 feeds the neuron update of the same step).  The barrier
// is a monotonic 64-bit arrival counter in global memory; every wait is bounded
// and a time-out sets an error flag and ends the kernel on all CTAs.
//
// Split delivery.  Only a synapse whose dendritic delay is zero steps (or a
// multiple of the ring length: it wraps around the ring) feeds the neuron update
// of the SAME step; for a typical cortical model that is a few per cent of the
// synapses.  The host copies exactly those into a small padded table per group
// ("urgent" synapses) and the step becomes
//
//   header    spike counts and ids of the step before
//   phase A0  urgent synapses of those spikes (+ every synapse of a group that
//             has no dendritic-delay ring)
//   barrier A
//   phase B   neuron update
//   barrier B arrive ... wait, and in between
//   phase A1  all OTHER synapses of the same spikes, same ring slots as always:
//             a slot one or more steps ahead is not read before the next neuron
//             update, and barrier A of the next step orders it.
//
// The bulk of the memory traffic thus overlaps the barrier (and, in a sharded
// model, the flight of the spike words between GPUs) instead of sitting on the
// critical path.  Results are those of the plain schedule: every contribution
// lands in the same slot before the same reader.
//
// One-step lag.  When EVERY synapse of every group has a dendritic delay of at
// least one step (the host scans the delay arrays), a spike emitted in step s
// may be delivered in the presynaptic phase of step s+2 instead of s+1, into
// the ring slot one position nearer: the value lands in the same slot before
// the neuron update that reads it, so the result is unchanged.  The spike lists
// a presynaptic phase reads were then completed before the PREVIOUS barrier, and
// the ring slots it writes are never the one a lagging CTA still reads, so the
// second barrier of the step disappears; in a sharded model the spike words
// have a whole step to cross NVLink.  The first pass of a launch has nothing to
// deliver (the launch before drained it) and one delivery pass runs after the
// last neuron update, so memory between launches is exactly what the two-barrier
// schedule leaves.
//
// Data written by other SMs between barriers (postsynaptic input, spike lists)
// is read with ld.global.cg so a stale L1 line can never be used.
#pragma once

#include "common.cuh"
#include "neuron_update.cuh"
#include "presynaptic_update.cuh"

namespace b200
{
struct NearRing;
struct NearSpace;
constexpr int FUSED_BLOCK = 768;          // one CTA per SM, 85 registers per thread
constexpr unsigned int FUSED_CHUNK = 32 * PRE_VEC;          // synapses per warp item
constexpr unsigned int FUSED_MAX_SOURCES = 256;             // (population, process, delay) spike sources per model
constexpr unsigned int FUSED_PREFETCH_IDS = 8;              // spike ids fetched together with each count
constexpr unsigned int ERR_BARRIER_TIMEOUT = 8u;
constexpr unsigned long long BARRIER_SPIN_LIMIT = 1ull << 24; // default: polls (tens of ms) before giving up

// One spike source as the presynaptic phase sees it: a (population, axonal
// delay) pair and the slice of the item table that lists every (group, chunk)
// a spike of this source has to visit.
struct FusedSource
{
    const unsigned int *spk_cnt;
    const unsigned int *spk;
    unsigned int num_src;
    unsigned int slots;
    unsigned int delay;
    unsigned int item_begin;             // items that may run after the neuron update (phase A1)
    unsigned int item_count;
    unsigned int urgent_begin;           // items that must run before it (phase A0)
    unsigned int urgent_count;
    unsigned int pad;
    const unsigned long long *spk_tag;   // sharded models: (step << 32 | count) per slot, else NULL
    const unsigned long long *spk_wire;  // sharded models: (step << 32 | id) lists, else NULL
};

// The urgent synapses of one SPARSE group, compressed rows.
struct FusedUrgent
{
    const unsigned int *offsets;         // [num_src + 1] into entries
    const uint2 *entries;                // (target index, weight bits)
    unsigned int stride;                 // longest row (0: the group has no urgent synapses)
    unsigned int pad;
};

// item.y of an urgent item: chunk index, with this bit set for a chunk of the
// urgent table (clear: a chunk of the full row of a group without delay ring)
constexpr unsigned int FUSED_URGENT_TABLE = 0x80000000u;

struct FusedLaunch
{
    NeuronLaunch neuron;                 // groups, batch(=1), dt, seed, recording, state
    const unsigned int *slot_start;      // [num_groups+1] first thread slot of each neuron group (multiples of 32)
    const b200_synapse_group *sgroups;
    const FusedSource *sources;
    const uint2 *items;                  // (synapse group index, chunk index); urgent items follow the others
    const FusedUrgent *urgent;           // [num_sgroups] or NULL (no group has an urgent table)
    unsigned int num_sources;
    unsigned int num_sgroups;
    unsigned int num_items;
    unsigned int stage_in_smem;          // tables fit the dynamic shared memory the host reserved
    unsigned int count_events;
    unsigned int profile;                // accumulate phase cycles (thread 0 of every CTA)
    unsigned long long *cta_cycles;      // [gridDim][4] or NULL
    unsigned long long num_steps;
    unsigned long long *barrier;         // monotonic arrival counter
    // spike exchange between the processes of a sharded model (world == 1: unused)
    unsigned int rank;
    unsigned int world;
    unsigned char *arena;                // this process's exchange arena
    unsigned char *const *peer_table;    // device table [B200_MAX_RANKS]: the same arena of every peer, mapped here
    unsigned int lag;                    // 1: deliver spikes one step late into the ring slot one nearer (see above)
    unsigned int skip_urgent;            // 1: full-row items leave out the synapses the urgent tables hold
    // warp-specialised kernel (stream_step.cuh) only
    unsigned int stream_warps;           // warps per CTA that do nothing but deliver non-urgent synapses
    unsigned int slots_per_cta;          // neuron slots per CTA (a multiple of 32)
    // "deliver at emission" mode of that kernel (near.cuh)
    unsigned int emit;                   // 1: the spiking thread delivers its near synapses, one barrier per step
    unsigned int num_rings;
    const struct NearRing *near_rings;   // [world][num_rings]: the rings of every process, as mapped here
    const struct NearSpace *near_spaces; // [neuron groups]
    // queues for near synapses onto other processes' neurons (near.cuh); queue_words == 0: reduce directly
    unsigned int publisher;              // 1: the block's last warp publishes the spike counts (sharded models)
    unsigned int queue_words;            // 64-bit words per queue, header included
    unsigned int queue_count;            // queues per (step parity, sending process)
    unsigned long long queue_offset;     // where the queues start in every process's arena
};

constexpr unsigned long long EXCHANGE_SPIN_LIMIT = 1ull << 23;  // default
constexpr unsigned int ERR_EXCHANGE_TIMEOUT = 32u;

__device__ __forceinline__ unsigned long long loadAcquireSys(const unsigned long long *p)
{
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ unsigned long long loadRelaxedSys(const unsigned long long *p)
{
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void storeRelaxedSys(unsigned long long *p, unsigned long long v)
{
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory");
}

// Poll a word written by another process into this process's memory until its
// high half is the step we expect.  Bounded; returns the low half (0 on time-out).
__device__ __forceinline__ unsigned int awaitWord(const unsigned long long *p, unsigned long long expected, StepState *state)
{
    unsigned long long w = 0, polls = 0;
    while(((w = loadRelaxedSys(p)) >> 32) != expected) {
        if(++polls > state->exchange_spin_limit) {
            atomicOr(&state->error, ERR_EXCHANGE_TIMEOUT);
            return 0u;
        }
    }
    return (unsigned int)w;
}

__device__ __forceinline__ unsigned long long loadAcquire(const unsigned long long *p)
{
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Grid-wide barrier in two halves so work that does not depend on other CTAs can
// run between them.  gridArrive publishes this CTA's writes and counts it in;
// gridWait blocks (bounded) until every CTA has arrived and returns false if it
// timed out, in which case every CTA leaves the kernel.
__device__ __forceinline__ void gridArrive(unsigned long long *barrier, unsigned long long &epoch)
{
    __syncthreads();
    if(threadIdx.x == 0) {
        // release + arrive in one fire-and-forget reduction: nothing waits for its return
        asm volatile("red.release.gpu.global.add.u64 [%0], %1;" :: "l"(barrier), "l"(1ull) : "memory");
    }
    epoch += gridDim.x;     // every thread keeps the count: any of them may have to poll
}

__device__ __forceinline__ bool gridWait(const unsigned long long *barrier, const unsigned long long &epoch, bool *ok,
                                         StepState *state)
{
    if(threadIdx.x == 0) {
        unsigned long long polls = 0;
        bool good = true;
        while(loadAcquire(barrier) < epoch) {
            if(++polls > state->barrier_spin_limit) {
                atomicOr(&state->error, ERR_BARRIER_TIMEOUT);
                good = false;
                break;
            }
        }
        *ok = good;
    }
    __syncthreads();
    return *ok;
}

template<typename IndT>
__device__ __forceinline__ void fusedChunk(const b200_synapse_group &g, unsigned int pre, unsigned int chunk,
                                           unsigned int front, unsigned int zeroDelay, StepState *state)
{
    const unsigned int D = g.max_den_delay;
    float *target = D ? g.den_delay : g.out_post;
    sparseQuad<IndT>(g, pre, chunk * 32u + (threadIdx.x & 31u), target, D ? ringSlot(front, D) : 0u, state, zeroDelay);
}

// 32 entries of one row of a group's urgent table into the front slot of its ring.
__device__ __forceinline__ void fusedUrgentChunk(const b200_synapse_group &g, const FusedUrgent &u, unsigned int pre,
                                                 unsigned int chunk, unsigned int front, StepState *state)
{
    const unsigned int begin = __ldg(&u.offsets[pre]), end = __ldg(&u.offsets[pre + 1]);
    const unsigned int at = begin + chunk * 32u + (threadIdx.x & 31u);
    if(at >= end) return;
    const uint2 e = __ldg(&u.entries[at]);
    if(e.x >= g.num_trg) {
        atomicOr(&state->error, ERR_IND_RANGE);
        return;
    }
    redAdd(g.den_delay + (unsigned long long)ringSlot(front, g.max_den_delay) * g.num_trg + e.x, __uint_as_float(e.y));
}

// Copy `bytes` (a multiple of 4) from global to shared memory with the whole CTA.
__device__ __forceinline__ void stageWords(void *dst, const void *src, size_t bytes)
{
    unsigned int *d = static_cast<unsigned int*>(dst);
    const unsigned int *s = static_cast<const unsigned int*>(src);
    for(size_t w = threadIdx.x; w < bytes / 4; w += blockDim.x) d[w] = __ldg(&s[w]);
}

__host__ __device__ inline size_t align16(size_t x) { return (x + 15) & ~(size_t)15; }

// The acquire side of every grid barrier invalidates the SM's L1, so a
// descriptor left in global memory would cost a full L2 round trip per field
// and per step, one after another along the dependency chain.  All merged-group
// tables are therefore staged into shared memory once per launch.
template<int NPSM, int NCS>
__global__ void __launch_bounds__(FUSED_BLOCK, 1)
fusedStepKernel(FusedLaunch L)
{
    extern __shared__ __align__(16) unsigned char fusedSmem[];
    __shared__ bool barrierOk;
    __shared__ long long publishedAt;        // profile mode: when the counts of the last step went out
    if(threadIdx.x == 0) publishedAt = 0;
    __shared__ unsigned int headCnt[FUSED_MAX_SOURCES], headSlot[FUSED_MAX_SOURCES], headIds[FUSED_MAX_SOURCES][FUSED_PREFETCH_IDS];
    __shared__ unsigned char *peerArena[B200_MAX_RANKS];
    if(threadIdx.x < B200_MAX_RANKS) peerArena[threadIdx.x] = L.peer_table ? L.peer_table[threadIdx.x] : nullptr;
    __shared__ ExchangeCtx exchange;
    if(threadIdx.x == 0) {
        exchange.world = L.world;
        exchange.rank = L.rank;
        exchange.arena = L.arena;
        exchange.peers = peerArena;
    }
    const ExchangeCtx *xp = (L.world > 1) ? &exchange : nullptr;
    if(L.stage_in_smem) {
        unsigned char *p = fusedSmem;
        const size_t nb = sizeof(b200_neuron_group) * L.neuron.num_groups;
        stageWords(p, L.neuron.groups, nb);
        L.neuron.groups = reinterpret_cast<const b200_neuron_group*>(p);
        p += align16(nb);
        const size_t sb = sizeof(b200_synapse_group) * L.num_sgroups;
        stageWords(p, L.sgroups, sb);
        L.sgroups = reinterpret_cast<const b200_synapse_group*>(p);
        p += align16(sb);
        const size_t rb = sizeof(FusedSource) * L.num_sources;
        stageWords(p, L.sources, rb);
        L.sources = reinterpret_cast<const FusedSource*>(p);
        p += align16(rb);
        const size_t ib = sizeof(uint2) * L.num_items;
        stageWords(p, L.items, ib);
        L.items = reinterpret_cast<const uint2*>(p);
        p += align16(ib);
        const size_t tb = sizeof(unsigned int) * (L.neuron.num_groups + 1);
        stageWords(p, L.slot_start, tb);
        L.slot_start = reinterpret_cast<const unsigned int*>(p);
        p += align16(tb);
        if(L.urgent) {
            stageWords(p, L.urgent, sizeof(FusedUrgent) * L.num_sgroups);
            L.urgent = reinterpret_cast<const FusedUrgent*>(p);
        }
        __syncthreads();
    }
    const unsigned int lane = threadIdx.x & 31u;
    const unsigned int warp = threadIdx.x >> 5;
    const unsigned int warpsPerBlock = blockDim.x >> 5;
    // work items go round-robin over CTAs first: a handful of items per step must
    // spread over every SM, because one SM retires scattered reductions slowly
    const unsigned int gwarp = (threadIdx.x >> 5) * gridDim.x + blockIdx.x;
    const unsigned int totalWarps = gridDim.x * warpsPerBlock;
    const unsigned int gthread = blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned int totalThreads = gridDim.x * blockDim.x;
    StepState *state = L.neuron.state;
    const unsigned int period = state->ring_period;
    unsigned int k = state->phase;
    const unsigned long long t0 = state->timestep;
    const unsigned long long done0 = state->steps_done;
    unsigned long long epoch = 0;        // the host zeroes the arrival counter before every launch
    const unsigned int numGroups = L.neuron.num_groups;
    const unsigned int totalSlots = L.slot_start[numGroups];

    // Register-resident neuron state: when every neuron slot has a thread of its
    // own, the thread keeps its neuron's variables in registers for the whole
    // launch and only the dendritic-delay front (and inputs that take reductions
    // directly) touch memory each step.
    const bool resident = totalSlots <= totalThreads;
    const bool mine = resident && gthread < totalSlots;
    unsigned int myGroup = 0, myLocal = 0;
    bool myActive = false;
    unsigned long long myIndex = 0;
    NeuronRegs<NPSM, NCS> regs;
    if(mine) {
        myGroup = findGroup(L.slot_start, numGroups, gthread);
        myLocal = gthread - L.slot_start[myGroup];
        const b200_neuron_group &g = L.neuron.groups[myGroup];
        myActive = myLocal < g.num_update;
        myIndex = g.first_neuron + myLocal;
        if(myActive) loadNeuron<true>(g, myIndex, regs);
    }

    const bool prof = L.profile && threadIdx.x == 0;
    long long c0 = 0, c1 = 0, c2 = 0, c3 = 0;
    const unsigned int lag = L.lag;
    // lists: one 64-bit store per (process, population) says "step s: n spikes"; it is
    // what the readers poll.  The ids already sit in every arena (stored as they were
    // emitted).  Called by the whole grid after a barrier that follows the emission.
    auto publishCounts = [&](unsigned int first, unsigned int writtenAt, unsigned long long tagStep) {
        // called by one warp (first = lane) of block 0
        for(unsigned int idx = first; L.world > 1 && blockIdx.x == 0 && idx < L.world * numGroups; idx += 32u) {
            const unsigned int peer = idx / numGroups, gi = idx - peer * numGroups;
            const b200_neuron_group &g = L.neuron.groups[gi];
            const unsigned int wslot = ringSlot(writtenAt, g.num_delay_slots);
            const unsigned long long tag = (tagStep << 32) | (unsigned long long)__ldcg(&g.spk_cnt[wslot]);
            unsigned long long *cell = reinterpret_cast<unsigned long long*>(&g.spk_tag[wslot]);
            if(peer != L.rank) {
                cell = reinterpret_cast<unsigned long long*>(peerArena[peer] + (reinterpret_cast<unsigned char*>(cell) - L.arena));
            }
            storeRelaxedSys(cell, tag);
        }
    };
    // Deliver the spikes the header holds through one of the two item lists of every source:
    // the items the coming neuron update needs, or the ones that can follow it.
    unsigned long long step = 0;
    auto deliver = [&](const bool urgentList) {
        for(unsigned int base = 0; base < L.num_sources; base += 32u) {
            const unsigned int cnt = (base + lane < L.num_sources) ? headCnt[base + lane] : 0u;
            const unsigned int per = (base + lane >= L.num_sources) ? 0u
                : urgentList ? L.sources[base + lane].urgent_count : L.sources[base + lane].item_count;
            unsigned int incl = cnt * per;
            #pragma unroll
            for(int o = 1; o < 32; o <<= 1) {
                const unsigned int v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if(lane >= o) incl += v;
            }
            const unsigned int total = __shfl_sync(0xFFFFFFFFu, incl, 31);
            for(unsigned int it = gwarp; it < total; it += totalWarps) {
                const unsigned int owner = __ffs(__ballot_sync(0xFFFFFFFFu, incl > it)) - 1u;
                const unsigned int ownIncl = __shfl_sync(0xFFFFFFFFu, incl, owner);
                const unsigned int ownPer = __shfl_sync(0xFFFFFFFFu, per, owner);
                const unsigned int ownCnt = headCnt[base + owner];
                const unsigned int rel = it - (ownIncl - ownCnt * ownPer);
                const unsigned int s = rel / ownPer;
                const unsigned int c = rel - s * ownPer;
                const FusedSource &src = L.sources[base + owner];
                unsigned int pre;
                if(s < FUSED_PREFETCH_IDS) {
                    pre = headIds[base + owner][s];
                }
                else if(src.spk_wire) {
                    const long long expected = (long long)(done0 + step) - (long long)(src.delay + lag);
                    pre = awaitWord(&src.spk_wire[(unsigned long long)headSlot[base + owner] * src.num_src + s],
                                    (unsigned long long)expected, state);
                }
                else {
                    pre = __ldcg(&src.spk[(unsigned long long)headSlot[base + owner] * src.num_src + s]);
                }
                const uint2 item = L.items[(urgentList ? src.urgent_begin : src.item_begin) + c];
                const b200_synapse_group &g = L.sgroups[item.x];
                if(pre < g.num_src) {
                    if(item.y & FUSED_URGENT_TABLE) {
                        fusedUrgentChunk(g, L.urgent[item.x], pre, item.y & ~FUSED_URGENT_TABLE, k + 1u, state);
                    }
                    else {
                        // synapses that arrive in the same step: delivered (plain schedule), an error
                        // (the schedule relies on there being none) or left to the group's urgent table
                        const unsigned int zeroDelay = urgentList ? 0u
                            : (L.skip_urgent && L.urgent && L.urgent[item.x].stride) ? 2u : 1u;
                        switch(g.ind_bytes) {
                        case 1: fusedChunk<uint8_t>(g, pre, item.y, k + 1u - lag, zeroDelay, state); break;
                        case 2: fusedChunk<uint16_t>(g, pre, item.y, k + 1u - lag, zeroDelay, state); break;
                        default: fusedChunk<uint32_t>(g, pre, item.y, k + 1u - lag, zeroDelay, state); break;
                        }
                        if(L.count_events && item.y == 0 && lane == 0) {
                            atomicAdd(&state->synaptic_events, (unsigned long long)__ldg(&g.row_length[pre]));
                        }
                    }
                }
                else if(lane == 0) {
                    atomicOr(&state->error, ERR_IND_RANGE);
                }
            }
        }
    };
    // with the one-step lag a last pass delivers what the final neuron update left pending
    const unsigned long long passes = L.num_steps + lag;
    for(step = 0; step < passes; step++) {
        if(prof) c0 = clock64();
        // probe 6: from the publication of the last step's counts to the start of this header
        if(prof && blockIdx.x == 0 && publishedAt) state->probe[6] += (unsigned long long)(c0 - publishedAt);
        const bool drain = (step == L.num_steps);
        // every CTA has to finish the last neuron update before its counts go out
        if(drain && L.world > 1) gridArrive(L.barrier, epoch);
        if(!lag || step > 0) {

        // ---------------- spike headers: counts and first ids of every source -----------------
        // A few warps of each CTA (one per 32 sources) fetch every source's spike count
        // together with its first spike ids and share them through shared memory.  If
        // every warp of the grid read these few words itself, the L2 slices holding them
        // would serialise thousands of requests.
        if(warp < (L.num_sources + 31u) / 32u) {
            const unsigned int si = warp * 32u + lane;
            unsigned int cnt = 0, rslot = 0;
            // all loads into registers first: a shared-memory store between two loads
            // through generic pointers would serialise them
            unsigned int ids[FUSED_PREFETCH_IDS];
            #pragma unroll
            for(unsigned int j = 0; j < FUSED_PREFETCH_IDS; j++) ids[j] = 0u;
            if(si < L.num_sources) {
                const FusedSource &src = L.sources[si];
                rslot = ringSlot(k + src.slots - src.delay - lag, src.slots);
                if(src.spk_tag) {
                    // Sharded model: count and ids are 64-bit words the list's owner wrote
                    // into THIS process's memory, each carrying the step it belongs to.
                    // Poll (bounded) until the count word of the step we need is there;
                    // the id words were sent long before it, so they are fetched together
                    // and only a word that is not there yet is polled for.
                    const long long expected = (long long)(done0 + step) - (long long)(src.delay + lag);
                    if(expected > 0) {
                        cnt = awaitWord(&src.spk_tag[rslot], (unsigned long long)expected, state);
                        // probe 4: header start to the count word of source 0 being there
                        if(prof && blockIdx.x == 0 && si == 0) state->probe[4] += (unsigned long long)(clock64() - c0);
                        const unsigned long long *wire = src.spk_wire + (unsigned long long)rslot * src.num_src;
                        unsigned long long words[FUSED_PREFETCH_IDS];
                        #pragma unroll
                        for(unsigned int j = 0; j < FUSED_PREFETCH_IDS; j++) words[j] = (j < cnt) ? loadRelaxedSys(&wire[j]) : 0ull;
                        #pragma unroll
                        for(unsigned int j = 0; j < FUSED_PREFETCH_IDS; j++) {
                            if(j < cnt) {
                                ids[j] = ((words[j] >> 32) == (unsigned long long)expected)
                                    ? (unsigned int)words[j] : awaitWord(&wire[j], (unsigned long long)expected, state);
                            }
                        }
                    }
                }
                else {
                    // fetched before the count is known: entries past the count are
                    // stale but valid memory
                    const unsigned int *list = src.spk + (unsigned long long)rslot * src.num_src;
                    cnt = __ldcg(&src.spk_cnt[rslot]);
                    #pragma unroll
                    for(unsigned int j = 0; j < FUSED_PREFETCH_IDS; j++) ids[j] = (j < src.num_src) ? __ldcg(&list[j]) : 0u;
                }
                #pragma unroll
                for(unsigned int j = 0; j < FUSED_PREFETCH_IDS; j++) headIds[si][j] = ids[j];
                headCnt[si] = cnt;
                headSlot[si] = rslot;
            }
        }
        __syncthreads();
        if(L.world > 1 && (__ldcg(&state->error) & ERR_EXCHANGE_TIMEOUT)) return;
        if(prof && L.cta_cycles) L.cta_cycles[4ull * gridDim.x + blockIdx.x] += (unsigned long long)(clock64() - c0);

        // ---------------- phase A (A0): what the coming neuron update needs ----------------
        if(lag) deliver(false);
        else deliver(true);
        }   // delivery pass
        if(drain) break;
        if(prof) c1 = clock64();
        if(L.world > 1 && threadIdx.x == 0) exchange.tag = done0 + step + 1;    // read after the barrier's __syncthreads
        gridArrive(L.barrier, epoch);
        // in the shadow of the barrier: this step's random draws
        unsigned int csCount[NCS > 0 ? NCS : 1] = {0};
        if(resident && mine && myActive) {
            drawCurrentSources<NCS>(L.neuron, L.neuron.groups[myGroup], 0u, (unsigned int)myIndex, t0 + step, csCount);
        }
        if(!gridWait(L.barrier, epoch, &barrierOk, state)) return;
        // lagging schedule: the lists of the step before are complete now
        if(lag && step > 0 && warp == 0) publishCounts(lane, k, done0 + step);
        if(prof) c2 = clock64();

        // ---------------- phase B: neuron update -----------------------------------
        if(resident) {
            if(mine) {
                const b200_neuron_group &g = L.neuron.groups[myGroup];
                const float t = B200_FMUL((float)(t0 + step), L.neuron.dt);
                bool spiked = false;
                if(myActive) {
                    float front[NPSM];
                    #pragma unroll
                    for(unsigned int p = 0; p < NPSM; p++) {
                        if(p < g.num_psm && !g.psm[p].max_den_delay) regs.lin[p] = __ldcg(&g.psm[p].out_post[myIndex]);
                    }
                    takeFronts<true, NPSM>(g, 0u, (unsigned int)myIndex, k, front);
                    spiked = neuronCompute(L.neuron, g, 0u, (unsigned int)myIndex, t0 + step, t, regs, front, csCount);
                    #pragma unroll
                    for(unsigned int p = 0; p < NPSM; p++) {
                        if(p < g.num_psm && !g.psm[p].max_den_delay) g.psm[p].out_post[myIndex] = regs.lin[p];
                    }
                }
                neuronEmit<true>(L.neuron, g, 0u, myLocal, spiked, k, t0 + step, t, xp);
            }
        }
        else {
            for(unsigned int slot = gthread; slot < totalSlots; slot += totalThreads) {
                const unsigned int gi = findGroup(L.slot_start, numGroups, slot);
                const b200_neuron_group &g = L.neuron.groups[gi];
                neuronStep<true, NPSM, NCS>(L.neuron, g, 0u, slot - L.slot_start[gi], k, t0 + step, xp);
            }
        }
        // spike-queue update for the next step (neuronUpdateGroupMerged.cc:947-975)
        if(gthread < numGroups) {
            const b200_neuron_group &o = L.neuron.groups[gthread];
            o.spk_cnt[ringSlot(k + 2, o.num_delay_slots)] = 0;
        }
        if(prof) c3 = clock64();
        if(!lag) {
            gridArrive(L.barrier, epoch);
            const long long arrivedAt = L.profile ? clock64() : 0;
            // sharded model: one warp waits for the last CTA and tells every process how many
            // spikes each population emitted; the readers poll those words, so nobody else
            // has to see the barrier complete before going on
            if(L.world > 1 && blockIdx.x == 0 && warp == warpsPerBlock - 1u) {
                unsigned long long polls = 0;
                while(loadAcquire(L.barrier) < epoch) {
                    if(++polls > state->barrier_spin_limit) {
                        atomicOr(&state->error, ERR_BARRIER_TIMEOUT);
                        break;
                    }
                }
                const long long seen = clock64();
                publishCounts(lane, k + 1u, done0 + step + 1);
                if(L.profile && lane == 0) {
                    // probe 0: this CTA's arrival to the barrier seen complete; probe 1: reading and sending the counts
                    const long long sent = clock64();
                    state->probe[0] += (unsigned long long)(seen - arrivedAt);
                    state->probe[1] += (unsigned long long)(sent - seen);
                    publishedAt = sent;
                }
            }
            // ---------------- phase A1: everything the next neuron update does not need ----------
            deliver(false);
            // probe 2: phase A1 on CTA 0; probe 3: what is left of the barrier after it
            const long long deliveredAt = prof ? clock64() : 0;
            if(!gridWait(L.barrier, epoch, &barrierOk, state)) return;
            if(prof && blockIdx.x == 0) {
                state->probe[2] += (unsigned long long)(deliveredAt - arrivedAt);
                state->probe[3] += (unsigned long long)(clock64() - deliveredAt);
            }
        }
        k = (k + 1 == period) ? 0u : k + 1;
        if(prof) {
            const long long c4 = clock64();
            if(blockIdx.x == 0) {
                state->phase_cycles[0] += (unsigned long long)(c1 - c0);
                state->phase_cycles[1] += (unsigned long long)(c2 - c1);
                state->phase_cycles[2] += (unsigned long long)(c3 - c2);
                state->phase_cycles[3] += (unsigned long long)(c4 - c3);
            }
            if(L.cta_cycles) {
                unsigned long long *mine4 = L.cta_cycles + 4ull * blockIdx.x;
                mine4[0] += (unsigned long long)(c1 - c0);
                mine4[1] += (unsigned long long)(c2 - c1);
                mine4[2] += (unsigned long long)(c3 - c2);
                mine4[3] += (unsigned long long)(c4 - c3);
            }
        }
    }
    if(lag && L.world > 1) {
        if(!gridWait(L.barrier, epoch, &barrierOk, state)) return;
        if(warp == 0) publishCounts(lane, k, done0 + L.num_steps);
    }
    if(mine && myActive) storeNeuron(L.neuron.groups[myGroup], myIndex, regs, true);
    if(gthread == 0) {
        state->timestep = t0 + L.num_steps;
        state->steps_done = state->steps_done + L.num_steps;
        state->phase = k;
    }
}
}   // namespace b200
