// Warp-specialised persistent time-step kernel.
//
// The step of a spiking network has a short dependent chain (neuron update ->
// spike lists -> the few synapses that arrive in the very next step -> neuron
// update) and a bulk of memory traffic that is NOT on it: every synapse with a
// dendritic delay of one step or more only has to land in its ring slot before
// the neuron update after next.  fusedStepKernel (fused_step.cuh) runs both on
// the same warps, so the bulk sits between the barriers of the chain.  Here the
// warps of every CTA are split:
//
//   chain warps  (the first C)   header -> urgent synapses -> grid barrier ->
//                                neuron update (state in registers) -> grid
//                                barrier.  Nothing else.
//   stream warps (the other S)   all remaining synapses of the spikes the chain
//                                warps announced, a whole step of time to do it:
//                                from the header of step s until the chain is
//                                about to pass the first barrier of step s+1.
//
// The two sets talk through shared memory only: the chain publishes the spike
// header of step s (double buffered) and a sequence number; each stream warp
// answers with the number of the last step whose deliveries it has made
// visible (__threadfence).  The chain's release at the grid barrier follows a
// read of those numbers, so the barrier orders the stream's reductions before
// the neuron update that reads them.
//
// What may be streamed and why the result is that of the plain schedule: see
// "Split delivery" in fused_step.cuh; the urgent tables are built by urgent.cuh.
#pragma once

#include "fused_step.cuh"
#include "near.cuh"

namespace b200
{
// Backstop for the waits between the two sets of warps (clock cycles, about half a minute): every
// wait of the other side is itself bounded and far shorter, so this only ends a CTA whose partner died.
constexpr long long STREAM_WAIT_CYCLES = 4000000000ll;   // default: about two seconds

// Barrier over the chain warps only (named barrier 1); the stream warps never join it.
__device__ __forceinline__ void chainSync(unsigned int chainThreads)
{
    asm volatile("bar.sync 1, %0;" :: "r"(chainThreads) : "memory");
}

struct StreamShared
{
    unsigned int headCnt[2][FUSED_MAX_SOURCES];
    unsigned int headSlot[2][FUSED_MAX_SOURCES];
    unsigned int headIds[2][FUSED_MAX_SOURCES][FUSED_PREFETCH_IDS];
    volatile unsigned int headReady;                 // steps whose header has been published
    volatile unsigned int stop;                      // the chain gave up: stream warps leave
    volatile unsigned int streamDone[32];            // per stream warp: steps fully delivered
    volatile unsigned int stepPassed;                // emit mode: grid barriers of the launch that have completed
    unsigned long long waited[2];                    // profile mode: cycles CTA 0 waited for the grid barrier / for the other processes
    volatile unsigned int streamGo[2];               // emit mode: the first stream warp's decision for a pass (pass number: go)
    bool barrierOk;
};

// Barrier over the stream warps only (named barrier 2).
__device__ __forceinline__ void streamSync(unsigned int streamThreads)
{
    asm volatile("bar.sync 2, %0;" :: "r"(streamThreads) : "memory");
}

// Spike count and first ids of source `si` for the step whose phase is `k` (`stepsDone` steps
// completed before it), into header buffer `buf`.  One lane per source.
__device__ __forceinline__ void fetchHeader(const FusedLaunch &L, StreamShared &sh, unsigned int buf, unsigned int si,
                                            unsigned int k, unsigned long long stepsDone, StepState *state)
{
    if(si >= L.num_sources) return;
    unsigned int cnt = 0;
    // all loads into registers first: a shared-memory store between two loads through generic
    // pointers would serialise them
    unsigned int ids[FUSED_PREFETCH_IDS];
    #pragma unroll
    for(unsigned int j = 0; j < FUSED_PREFETCH_IDS; j++) ids[j] = 0u;
    const FusedSource &src = L.sources[si];
    const unsigned int rslot = ringSlot(k + src.slots - src.delay, src.slots);
    if(src.spk_tag) {
        // sharded model: (step, count) and (step, id) words written by the list's owner into THIS
        // process's memory; poll (bounded) for the count of the step we need
        const long long expected = (long long)stepsDone - (long long)src.delay;
        if(expected > 0) {
            cnt = awaitWord(&src.spk_tag[rslot], (unsigned long long)expected, state);
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
        // ids fetched before the count is known: entries past it are stale but valid memory
        const unsigned int *list = src.spk + (unsigned long long)rslot * src.num_src;
        cnt = __ldcg(&src.spk_cnt[rslot]);
        #pragma unroll
        for(unsigned int j = 0; j < FUSED_PREFETCH_IDS; j++) ids[j] = (j < src.num_src) ? __ldcg(&list[j]) : 0u;
    }
    #pragma unroll
    for(unsigned int j = 0; j < FUSED_PREFETCH_IDS; j++) sh.headIds[buf][si][j] = ids[j];
    sh.headCnt[buf][si] = cnt;
    sh.headSlot[buf][si] = rslot;
}

// One pass over one of the two item lists of every source, for the spikes whose
// header sits in buffer `buf`: warp `first` of `stride` takes every stride-th item.
__device__ __forceinline__ void deliverItems(const FusedLaunch &L, const StreamShared &sh, unsigned int buf,
                                             bool urgentList, unsigned int first, unsigned int stride,
                                             unsigned int k, unsigned long long stepsDone, StepState *state,
                                             int farMode = -1)
{
    const unsigned int lane = threadIdx.x & 31u;
    for(unsigned int base = 0; base < L.num_sources; base += 32u) {
        const unsigned int cnt = (base + lane < L.num_sources) ? sh.headCnt[buf][base + lane] : 0u;
        const unsigned int per = (base + lane >= L.num_sources) ? 0u
            : urgentList ? L.sources[base + lane].urgent_count : L.sources[base + lane].item_count;
        unsigned int incl = cnt * per;
        #pragma unroll
        for(int o = 1; o < 32; o <<= 1) {
            const unsigned int v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if(lane >= o) incl += v;
        }
        const unsigned int total = __shfl_sync(0xFFFFFFFFu, incl, 31);
        for(unsigned int it = first; it < total; it += stride) {
            const unsigned int owner = __ffs(__ballot_sync(0xFFFFFFFFu, incl > it)) - 1u;
            const unsigned int ownIncl = __shfl_sync(0xFFFFFFFFu, incl, owner);
            const unsigned int ownPer = __shfl_sync(0xFFFFFFFFu, per, owner);
            const unsigned int ownCnt = sh.headCnt[buf][base + owner];
            const unsigned int rel = it - (ownIncl - ownCnt * ownPer);
            const unsigned int s = rel / ownPer;
            const unsigned int c = rel - s * ownPer;
            const FusedSource &src = L.sources[base + owner];
            unsigned int pre;
            if(s < FUSED_PREFETCH_IDS) {
                pre = sh.headIds[buf][base + owner][s];
            }
            else if(src.spk_wire) {
                const long long expected = (long long)stepsDone - (long long)src.delay;
                pre = awaitWord(&src.spk_wire[(unsigned long long)sh.headSlot[buf][base + owner] * src.num_src + s],
                                (unsigned long long)expected, state);
            }
            else {
                pre = __ldcg(&src.spk[(unsigned long long)sh.headSlot[buf][base + owner] * src.num_src + s]);
            }
            const uint2 item = L.items[(urgentList ? src.urgent_begin : src.item_begin) + c];
            const b200_synapse_group &g = L.sgroups[item.x];
            if(pre < g.num_src) {
                if(item.y & FUSED_URGENT_TABLE) {
                    fusedUrgentChunk(g, L.urgent[item.x], pre, item.y & ~FUSED_URGENT_TABLE, k + 1u, state);
                }
                else {
                    // a synapse that arrives in the same step: delivered here (urgent list), in the
                    // group's urgent table (skipped here), or an error (no table: none may exist)
                    // (farMode overrides: 0 deliver every synapse, 3 leave out delays 0 and 1)
                    const unsigned int zeroDelay = (farMode >= 0) ? (unsigned int)farMode
                        : urgentList ? 0u : (L.urgent && L.urgent[item.x].stride) ? 2u : 1u;
                    switch(g.ind_bytes) {
                    case 1: fusedChunk<uint8_t>(g, pre, item.y, k + 1u, zeroDelay, state); break;
                    case 2: fusedChunk<uint16_t>(g, pre, item.y, k + 1u, zeroDelay, state); break;
                    default: fusedChunk<uint32_t>(g, pre, item.y, k + 1u, zeroDelay, state); break;
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
}

// What one lane holds of one (spike, 128-synapse chunk) item between its loads and its reductions.
struct StreamQuad
{
    unsigned int group;          // index of the synapse group, 0xFFFFFFFF: nothing to do
    unsigned int pre;
    unsigned int len;
    unsigned int post[4];
    float w[4];
    unsigned int dw;             // four delays
    unsigned long long idx;      // index of the quad's first synapse in the group's arrays
};

__device__ __forceinline__ void streamQuadLoad(const b200_synapse_group &g, unsigned int pre, unsigned int quad, StreamQuad &q)
{
    const unsigned long long rowStart = (unsigned long long)pre * g.row_stride;
    q.idx = (rowStart & ~3ull) + (unsigned long long)quad * PRE_VEC;
    q.pre = pre;
    if(q.idx >= (unsigned long long)g.num_src * g.row_stride) {
        q.group = 0xFFFFFFFFu;
        return;
    }
    // row length and row data together: the quad's address does not depend on the length, and a
    // quad past the end of its row still lies inside the array (or its tail padding)
    q.len = __ldg(&g.row_length[pre]);
    switch(g.ind_bytes) {
    case 1: IndLoad<uint8_t>::load4(g.ind, q.idx, q.post); break;
    case 2: IndLoad<uint16_t>::load4(g.ind, q.idx, q.post); break;
    default: IndLoad<uint32_t>::load4(g.ind, q.idx, q.post); break;
    }
    if(g.wu_model == B200_WU_STATIC_PULSE_CONSTANT_WEIGHT) {
        q.w[0] = q.w[1] = q.w[2] = q.w[3] = g.wu_params[0];
    }
    else {
        const float4 wv = __ldg(reinterpret_cast<const float4*>(g.g + q.idx));
        q.w[0] = wv.x; q.w[1] = wv.y; q.w[2] = wv.z; q.w[3] = wv.w;
    }
    q.dw = g.max_den_delay ? __ldg(reinterpret_cast<const unsigned int*>(g.d + q.idx)) : 0u;
}

// The reductions of a loaded quad; `zeroDelay` as in sparseQuad.
__device__ __forceinline__ void streamQuadApply(const b200_synapse_group &g, const StreamQuad &q, unsigned int front,
                                                unsigned int zeroDelay, StepState *state)
{
    const unsigned long long rowStart = (unsigned long long)q.pre * g.row_stride;
    const unsigned long long rowEnd = rowStart + q.len;
    const unsigned int D = g.max_den_delay, numTrg = g.num_trg;
    float *target = D ? g.den_delay : g.out_post;
    const unsigned int denFront = D ? ringSlot(front, D) : 0u;
    #pragma unroll
    for(int j = 0; j < PRE_VEC; j++) {
        const unsigned long long sIdx = q.idx + j;
        if(sIdx >= rowStart && sIdx < rowEnd) {
            const unsigned int p = q.post[j];
            if(p >= numTrg) {
                atomicOr(&state->error, ERR_IND_RANGE);
                continue;
            }
            if(D) {
                unsigned int slot = denFront + ((q.dw >> (8 * j)) & 0xFFu);
                while(slot >= D) slot -= D;
                if(zeroDelay) {
                    if(slot == denFront) {
                        if(zeroDelay == 1u) atomicOr(&state->error, ERR_DELAY_RANGE);
                        continue;
                    }
                    if(zeroDelay == 3u && slot == ((denFront + 1u == D) ? 0u : denFront + 1u)) continue;
                }
                redAdd(target + (unsigned long long)slot * numTrg + p, q.w[j]);
            }
            else {
                redAdd(target + p, q.w[j]);
            }
        }
    }
}

constexpr unsigned int STREAM_BATCH = 2;     // items a stream warp keeps in flight

// deliverItems for the stream warps: the same items, STREAM_BATCH at a time with the loads of all
// of them issued before the first reduction (a stream warp is bound by memory latency, and there
// are only a few of them per SM).  Full-row items only.
__device__ __forceinline__ void streamItems(const FusedLaunch &L, const StreamShared &sh, unsigned int buf,
                                            unsigned int first, unsigned int stride, unsigned int k,
                                            unsigned long long stepsDone, StepState *state, int farMode)
{
    const unsigned int lane = threadIdx.x & 31u;
    for(unsigned int base = 0; base < L.num_sources; base += 32u) {
        const unsigned int cnt = (base + lane < L.num_sources) ? sh.headCnt[buf][base + lane] : 0u;
        const unsigned int per = (base + lane >= L.num_sources) ? 0u : L.sources[base + lane].item_count;
        unsigned int incl = cnt * per;
        #pragma unroll
        for(int o = 1; o < 32; o <<= 1) {
            const unsigned int v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if(lane >= o) incl += v;
        }
        const unsigned int total = __shfl_sync(0xFFFFFFFFu, incl, 31);
        for(unsigned int it0 = first; it0 < total; it0 += stride * STREAM_BATCH) {
            StreamQuad q[STREAM_BATCH];
            #pragma unroll
            for(unsigned int u = 0; u < STREAM_BATCH; u++) {
                const unsigned int it = it0 + u * stride;
                q[u].group = 0xFFFFFFFFu;
                if(it >= total) continue;                       // the same for every lane
                const unsigned int owner = __ffs(__ballot_sync(0xFFFFFFFFu, incl > it)) - 1u;
                const unsigned int ownIncl = __shfl_sync(0xFFFFFFFFu, incl, owner);
                const unsigned int ownPer = __shfl_sync(0xFFFFFFFFu, per, owner);
                const unsigned int ownCnt = sh.headCnt[buf][base + owner];
                const unsigned int rel = it - (ownIncl - ownCnt * ownPer);
                const unsigned int sp = rel / ownPer;
                const unsigned int c = rel - sp * ownPer;
                const FusedSource &src = L.sources[base + owner];
                unsigned int pre;
                if(sp < FUSED_PREFETCH_IDS) {
                    pre = sh.headIds[buf][base + owner][sp];
                }
                else if(src.spk_wire) {
                    const long long expected = (long long)stepsDone - (long long)src.delay;
                    pre = awaitWord(&src.spk_wire[(unsigned long long)sh.headSlot[buf][base + owner] * src.num_src + sp],
                                    (unsigned long long)expected, state);
                }
                else {
                    pre = __ldcg(&src.spk[(unsigned long long)sh.headSlot[buf][base + owner] * src.num_src + sp]);
                }
                const uint2 item = L.items[src.item_begin + c];
                const b200_synapse_group &g = L.sgroups[item.x];
                if(pre >= g.num_src) {
                    if(lane == 0) atomicOr(&state->error, ERR_IND_RANGE);
                    continue;
                }
                q[u].group = item.x;
                streamQuadLoad(g, pre, item.y * 32u + lane, q[u]);
                if(L.count_events && item.y == 0 && lane == 0) {
                    atomicAdd(&state->synaptic_events, (unsigned long long)__ldg(&g.row_length[pre]));
                }
            }
            #pragma unroll
            for(unsigned int u = 0; u < STREAM_BATCH; u++) {
                if(q[u].group == 0xFFFFFFFFu) continue;
                const unsigned int zeroDelay = (farMode >= 0) ? (unsigned int)farMode
                    : (L.urgent && L.urgent[q[u].group].stride) ? 2u : 1u;
                streamQuadApply(L.sgroups[q[u].group], q[u], k + 1u, zeroDelay, state);
            }
        }
    }
}

// SHARDED: the model is spread over several processes (spike exchange, count words, waiting for the other
// processes).  A separate instance, so that one process pays for none of it on its critical path.
template<int NPSM, int NCS, bool SHARDED>
__global__ void __launch_bounds__(FUSED_BLOCK, 1)
streamStepKernel(FusedLaunch L)
{
    if(!SHARDED) L.world = 1u;
    extern __shared__ __align__(16) unsigned char fusedSmem[];
    __shared__ StreamShared sh;
    __shared__ unsigned char *peerArena[B200_MAX_RANKS];
    __shared__ ExchangeCtx exchange;
    __shared__ NearOutbox outbox;
    if(threadIdx.x < B200_MAX_RANKS) {
        peerArena[threadIdx.x] = L.peer_table ? L.peer_table[threadIdx.x] : nullptr;
        // this CTA's queue (step parity 0) in the arena of process threadIdx.x: written by this process, so
        // in the section of L.rank there
        unsigned char *base = (threadIdx.x == L.rank) ? L.arena : peerArena[threadIdx.x];
        outbox.queue[threadIdx.x] = (SHARDED && L.queue_words && base && blockIdx.x < L.queue_count)
            ? reinterpret_cast<unsigned long long*>(base + L.queue_offset) +
              ((unsigned long long)L.rank * L.queue_count + blockIdx.x) * L.queue_words
            : nullptr;
        outbox.count[threadIdx.x] = 0u;
    }
    if(threadIdx.x == 0) {
        outbox.words = (SHARDED && L.emit && L.world > 1 && blockIdx.x < L.queue_count) ? L.queue_words : 0u;
        outbox.fenced = 0u;
        outbox.parity_words = (unsigned long long)L.world * L.queue_count * L.queue_words;
    }
    if(threadIdx.x < 32) sh.streamDone[threadIdx.x] = 0u;
    if(threadIdx.x == 0) {
        exchange.world = L.world;
        exchange.rank = L.rank;
        exchange.arena = L.arena;
        exchange.peers = peerArena;
        sh.headReady = 0u;
        sh.stop = 0u;
        exchange.tag = L.neuron.state->steps_done + 1;     // emit mode: tag of the first step's spike words
    }
    const ExchangeCtx *xp = (SHARDED && L.world > 1) ? &exchange : nullptr;
    {
        // all merged-group tables into shared memory (the host made sure they fit): the acquire
        // side of a grid barrier invalidates L1, so descriptors in global memory would cost an
        // L2 round trip per field and step
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
            p += align16(sizeof(FusedUrgent) * L.num_sgroups);
        }
        if(L.emit) {
            stageWords(p, L.near_rings, sizeof(NearRing) * L.num_rings * L.world);
            L.near_rings = reinterpret_cast<const NearRing*>(p);
            p += align16(sizeof(NearRing) * L.num_rings * L.world);
            stageWords(p, L.near_spaces, sizeof(NearSpace) * L.neuron.num_groups);
            L.near_spaces = reinterpret_cast<const NearSpace*>(p);
        }
    }
    if(threadIdx.x == 0) sh.stepPassed = 0u;
    __syncthreads();        // the last barrier every warp of the CTA takes part in

    const unsigned int lane = threadIdx.x & 31u;
    const unsigned int warp = threadIdx.x >> 5;
    const unsigned int warpsPerBlock = blockDim.x >> 5;
    const unsigned int streamWarps = L.stream_warps;
    // (sharded model: the last warp of the block is neither: in CTA 0 it tells the other processes the spike
    // counts of every step the moment the step's barrier completes, off every other warp's path)
    const unsigned int publisherWarps = (SHARDED && L.world > 1 && L.publisher) ? 1u : 0u;
    const unsigned int chainWarps = warpsPerBlock - streamWarps - publisherWarps;
    const unsigned int chainThreads = chainWarps * 32u;
    StepState *state = L.neuron.state;
    const unsigned int period = state->ring_period;
    unsigned int k = state->phase;
    const unsigned long long t0 = state->timestep;
    const unsigned long long done0 = state->steps_done;

    // =========================== publisher warp ================================================
    if(publisherWarps && warp == warpsPerBlock - 1u) {
        if(blockIdx.x != 0) return;
        // "step s: n spikes", one 64-bit store per process and population, once the barrier behind the
        // neuron update of that step has completed (emit schedule: barrier number step + 2 of the launch,
        // the first one ends the prologue; otherwise two barriers per step); the ids already sit in every arena
        const unsigned int numGroups = L.neuron.num_groups;
        for(unsigned long long step = 0; step < L.num_steps; step++) {
            const unsigned long long target = (unsigned long long)gridDim.x * (L.emit ? step + 2ull : 2ull * step + 2ull);
            bool good = true;
            if(lane == 0) {
                unsigned long long polls = 0;
                while(loadAcquire(L.barrier) < target) {
                    if(sh.stop || ++polls > state->barrier_spin_limit) { good = false; break; }
                    __nanosleep(64);
                }
            }
            if(!__shfl_sync(0xFFFFFFFFu, good ? 1u : 0u, 0)) return;
            for(unsigned int idx = lane; idx < L.world * numGroups; idx += 32u) {
                const unsigned int peer = idx / numGroups, gi = idx - peer * numGroups;
                const b200_neuron_group &g = L.neuron.groups[gi];
                const unsigned int wslot = ringSlot(k + 1u, g.num_delay_slots);
                const unsigned long long tag = ((done0 + step + 1) << 32) | (unsigned long long)__ldcg(&g.spk_cnt[wslot]);
                unsigned long long *cell = reinterpret_cast<unsigned long long*>(&g.spk_tag[wslot]);
                if(peer != L.rank) {
                    cell = reinterpret_cast<unsigned long long*>(peerArena[peer] + (reinterpret_cast<unsigned char*>(cell) - L.arena));
                }
                storeRelaxedSys(cell, tag);
            }
            k = (k + 1 == period) ? 0u : k + 1;
        }
        return;
    }

    // =========================== stream warps ==================================================
    if(warp >= chainWarps && L.emit) {
        // Emit mode.  The spikes of launch step c-1 (c = 1 .. steps-1) are complete once the grid
        // barrier that ends that step has been passed; a pass of the stream warps fetches their
        // header and delivers every synapse with a delay of two steps or more, as the presynaptic
        // phase of step c would.  The chain waits for pass c before it arrives at the barrier that
        // ends step c+1: a pass has two steps of time.  One item costs several thousand cycles
        // (a few hundred dependent instructions around a random row), more than a step, so the stream
        // warps form two sets that take the odd and the even passes: a pass starts the moment its
        // spikes are there.  The sets are the CTAs with odd and with even index: equal halves of the
        // grid, and every stream warp of a CTA serves the same pass.
        const unsigned int me = warp - chainWarps;
        const bool alone = gridDim.x < 2u;                                 // a single CTA serves every pass
        const unsigned int set = blockIdx.x & 1u;
        const unsigned int setCtas = alone ? 1u : (gridDim.x + 1u - set) / 2u;     // CTAs set, set + 2, ...
        const unsigned int setThreads = streamWarps * 32u;
        const unsigned int first = me * setCtas + (blockIdx.x >> 1), stride = streamWarps * setCtas;
        unsigned long long spent[4] = {0, 0, 0, 0};     // profile mode: waiting, header, items, fence
        // passes c with c % 2 == set; phase of step c
        unsigned long long c = (set || alone) ? 1ull : 2ull;
        for(unsigned int a = 0; a < (unsigned int)c; a++) k = (k + 1 == period) ? 0u : k + 1;
        for(; c < L.num_steps; c += alone ? 1 : 2) {
            const long long since = clock64();
            bool alive = true;
            while(sh.stepPassed < (unsigned int)c) {
                if(sh.stop || clock64() - since > state->stream_wait_cycles) { alive = false; break; }
                __nanosleep(200);
            }
            // go on or leave TOGETHER (a warp that left alone would hang the others of its set on their
            // barrier): the set's first warp decides, the others read its decision behind the barrier
            const unsigned int buf = (unsigned int)(c & 1u);
            const long long t1 = clock64();
            if(me == 0 && lane == 0) sh.streamGo[buf] = (alive && !sh.stop) ? (unsigned int)c : 0u;
            __threadfence_block();
            for(unsigned int si = me * 32u + lane; si < ((L.num_sources + 31u) & ~31u); si += setThreads) {
                fetchHeader(L, sh, buf, si, k, done0 + c, state);
            }
            streamSync(setThreads);
            if(sh.streamGo[buf] != (unsigned int)c) return;
            const long long t2 = clock64();
            streamItems(L, sh, buf, first, stride, k, done0 + c, state, 3);
            const long long t3 = clock64();
            __threadfence();
            __syncwarp();
            if(lane == 0) sh.streamDone[me] = (unsigned int)c;
            k = (k + 1 == period) ? 0u : k + 1;
            if(!alone) k = (k + 1 == period) ? 0u : k + 1;
            spent[0] += (unsigned long long)(t1 - since);
            spent[1] += (unsigned long long)(t2 - t1);
            spent[2] += (unsigned long long)(t3 - t2);
            spent[3] += (unsigned long long)(clock64() - t3);
        }
        if(L.profile && blockIdx.x == 1 && me == 0 && lane == 0) {
            state->probe[0] += spent[0];
            state->probe[1] += spent[1];
            state->probe[3] += spent[2];
            state->probe[4] += spent[3];
        }
        return;
    }
    if(warp >= chainWarps) {
        const unsigned int me = warp - chainWarps;
        const unsigned int first = me * gridDim.x + blockIdx.x, stride = streamWarps * gridDim.x;
        unsigned long long busy = 0, idle = 0;
        for(unsigned long long step = 0; step < L.num_steps; step++) {
            const long long since = clock64();
            while(sh.headReady < (unsigned int)(step + 1)) {
                if(sh.stop) return;
                if(clock64() - since > state->stream_wait_cycles) {
                    if(lane == 0) atomicOr(&state->error, ERR_BARRIER_TIMEOUT);
                    return;
                }
                __nanosleep(200);
            }
            __threadfence_block();
            __syncwarp();
            const long long began = clock64();
            streamItems(L, sh, (unsigned int)(step & 1u), first, stride, k, done0 + step, state, -1);
            // reductions of every lane visible device-wide, then say so
            __threadfence();
            __syncwarp();
            if(lane == 0) sh.streamDone[me] = (unsigned int)(step + 1);
            k = (k + 1 == period) ? 0u : k + 1;
            idle += (unsigned long long)(began - since);
            busy += (unsigned long long)(clock64() - began);
        }
        // profile mode: probe 0/1 = cycles the first stream warp of CTA 0 spent waiting for a header / delivering
        if(L.profile && blockIdx.x == 0 && me == 0 && lane == 0) {
            state->probe[0] += idle;
            state->probe[1] += busy;
        }
        return;
    }

    // =========================== chain warps ===================================================
    unsigned long long epoch = 0;        // the host zeroes the arrival counter before every launch
    const unsigned int numGroups = L.neuron.num_groups;
    const unsigned int totalSlots = L.slot_start[numGroups];
    // neuron slots are dealt out evenly: slots_per_cta (a multiple of 32, at most the chain's
    // threads) to every CTA, one neuron per thread, state in registers for the whole launch
    const unsigned int slot = blockIdx.x * L.slots_per_cta + threadIdx.x;
    const bool mine = threadIdx.x < L.slots_per_cta && slot < totalSlots;
    unsigned int myGroup = 0, myLocal = 0;
    bool myActive = false;
    unsigned long long myIndex = 0;
    NeuronRegs<NPSM, NCS> regs;
    if(mine) {
        myGroup = findGroup(L.slot_start, numGroups, slot);
        myLocal = slot - L.slot_start[myGroup];
        const b200_neuron_group &g = L.neuron.groups[myGroup];
        myActive = myLocal < g.num_update;
        myIndex = g.first_neuron + myLocal;
        if(myActive) loadNeuron<true>(g, myIndex, regs);
    }
    const unsigned int chainFirst = warp * gridDim.x + blockIdx.x, chainStride = chainWarps * gridDim.x;

    // leave, taking the stream warps along
    #define B200_CHAIN_ABORT() do { sh.stop = 1u; return; } while(0)

    const bool prof = L.profile && threadIdx.x == 0;
    if(threadIdx.x == 0) { sh.waited[0] = 0; sh.waited[1] = 0; }
    auto arrive = [&]() {
        chainSync(chainThreads);
        if(threadIdx.x == 0) {
            asm volatile("red.release.gpu.global.add.u64 [%0], %1;" :: "l"(L.barrier), "l"(1ull) : "memory");
        }
        epoch += gridDim.x;
    };
    // `peersAt`: if not zero, also wait until every other process has announced that step (its count
    // word of the first population, in queue slot `peersSlot`, carries the step): everything it sent before that, the
    // reductions of its near synapses into THIS process's rings included, has landed.
    auto wait = [&](unsigned long long peersAt = 0ull, unsigned int peersSlot = 0u) -> bool {
        if(warp == 0) {
            bool good = true;
            const long long w0 = prof ? clock64() : 0;
            // the error word travels while the barrier is being polled (sticky bits: a flag raised after this
            // load is seen one step later)
            unsigned int seen = 0;
            if(lane == 0) {
                seen = __ldcg(&state->error);
                unsigned long long polls = 0;
                while(loadAcquire(L.barrier) < epoch) {
                    if(++polls > state->barrier_spin_limit) {
                        atomicOr(&state->error, ERR_BARRIER_TIMEOUT);
                        good = false;
                        break;
                    }
                }
            }
            good = __shfl_sync(0xFFFFFFFFu, good ? 1u : 0u, 0) != 0u;
            const long long w1 = prof ? clock64() : 0;
            if(SHARDED && good && peersAt && lane < L.world && lane != L.rank) {
                // the sections of a population's count words lie one process after the other; this
                // process's own pointer is in its descriptor
                const b200_neuron_group &g0 = L.neuron.groups[0];
                const unsigned long long *word = reinterpret_cast<const unsigned long long*>(g0.spk_tag) +
                    ((long long)lane - (long long)L.rank) * (long long)g0.num_delay_slots + peersSlot;
                unsigned long long polls = 0;
                while((loadRelaxedSys(word) >> 32) != peersAt) {
                    if(++polls > state->exchange_spin_limit) {
                        atomicOr(&state->error, ERR_EXCHANGE_TIMEOUT);
                        break;
                    }
                }
            }
            __syncwarp();
            if(prof) {      // probe 5: this CTA's wait for the grid barrier, probe 6: for the other processes
                sh.waited[0] += (unsigned long long)(w1 - w0);
                sh.waited[1] += (unsigned long long)(clock64() - w1);
            }
            // one thread decides for all: a CTA whose chain threads disagreed would hang on its barrier
            if(lane == 0) {
                if(seen & (ERR_BARRIER_TIMEOUT | ERR_EXCHANGE_TIMEOUT)) good = false;
                sh.barrierOk = good;
            }
        }
        chainSync(chainThreads);
        return sh.barrierOk;
    };

    long long c0 = 0, c1 = 0, c2 = 0, c3 = 0;
    unsigned long long cyc[6] = {0, 0, 0, 0, 0, 0};
    const bool emit = L.emit != 0;
    unsigned int csCount[NCS > 0 ? NCS : 1] = {0};
    if(emit) {
        // The spikes of the step before this launch: every synapse of theirs, as the plain schedule's
        // presynaptic phase would deliver them, then a grid barrier.  (The last step of a launch leaves
        // its spikes undelivered, so that memory between launches is what every other path expects.)
        if(warp < (L.num_sources + 31u) / 32u) fetchHeader(L, sh, 0u, warp * 32u + lane, k, done0, state);
        chainSync(chainThreads);
        deliverItems(L, sh, 0u, false, chainFirst, chainStride, k, done0, state, 0);
        arrive();
        if(mine && myActive) {
            drawCurrentSources<NCS>(L.neuron, L.neuron.groups[myGroup], 0u, (unsigned int)myIndex, t0, csCount);
        }
        if(!wait()) B200_CHAIN_ABORT();
    }
    for(unsigned long long step = 0; step < L.num_steps; step++) {
        if(prof) c0 = clock64();
        const unsigned int buf = (unsigned int)(step & 1u);
        if(emit) {
            if(prof) { c1 = clock64(); c2 = c1; }
        }
        else {

        // ---------------- header: spike counts and first ids of every source ----------------------
        if(warp < (L.num_sources + 31u) / 32u) fetchHeader(L, sh, buf, warp * 32u + lane, k, done0 + step, state);
        chainSync(chainThreads);
        if(threadIdx.x == 0) {
            __threadfence_block();
            sh.headReady = (unsigned int)(step + 1);        // the stream warps start on this step
        }
        if(prof) cyc[4] += (unsigned long long)(clock64() - c0);

        // ---------------- phase A0: what the coming neuron update needs ---------------------------
        deliverItems(L, sh, buf, true, chainFirst, chainStride, k, done0 + step, state);
        if(prof) c1 = clock64();

        // the stream warps must have delivered the spikes of the step before: the slot the coming
        // neuron update reads may hold their contributions
        if(threadIdx.x == 0 && step > 0) {
            const long long since = clock64();
            if(prof) c1 = since;
            for(unsigned int w = 0; w < streamWarps; w++) {
                while(sh.streamDone[w] < (unsigned int)step) {
                    if(clock64() - since > state->stream_wait_cycles) {
                        atomicOr(&state->error, ERR_BARRIER_TIMEOUT);
                        break;
                    }
                }
            }
            // (no fence of its own: the release at the barrier below follows in program order and is
            // cumulative over what this thread has just observed)
            if(prof) cyc[5] += (unsigned long long)(clock64() - since);
        }
        if(SHARDED && L.world > 1 && threadIdx.x == 0) exchange.tag = done0 + step + 1;    // read after the barrier below
        arrive();
        // in the shadow of the barrier: this step's random draws
        if(mine && myActive) {
            drawCurrentSources<NCS>(L.neuron, L.neuron.groups[myGroup], 0u, (unsigned int)myIndex, t0 + step, csCount);
        }
        if(!wait()) B200_CHAIN_ABORT();
        if(prof) c2 = clock64();
        }   // header, urgent synapses and first barrier (not in emit mode)

        // ---------------- phase B: neuron update ----------------------------------------------
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
            if(emit && step + 1 < L.num_steps) {
                // the near rows of this warp's spiking neurons are needed in a moment: start them on
                // their way into L2 while the spike lists are being written (an atomic round trip)
                unsigned int ahead = __ballot_sync(0xFFFFFFFFu, spiked);
                const NearSpace space = L.near_spaces[myGroup];
                while(ahead && space.shift != 0xFFFFFFFFu) {
                    const unsigned int b = __ffs(ahead) - 1u;
                    ahead &= ahead - 1u;
                    const unsigned int id = __shfl_sync(0xFFFFFFFFu, (unsigned int)myIndex, b);
                    if((lane << 4) < (1u << space.shift)) {         // one 128-byte line (16 entries) per lane
                        const uint2 *line = space.rows + ((unsigned long long)(id - space.first_row) << space.shift) + (lane << 4);
                        asm volatile("prefetch.global.L2 [%0];" :: "l"(line));
                    }
                }
            }
            neuronEmit<true>(L.neuron, g, 0u, myLocal, spiked, k, t0 + step, t, xp);
            if(emit && step + 1 < L.num_steps) {
                // the warp delivers the near synapses of its spiking neurons, one row after the other
                unsigned int ballot = __ballot_sync(0xFFFFFFFFu, spiked);
                float returned = 0.0f;
                const NearSpace space = L.near_spaces[myGroup];
                const bool timeIt = L.profile && ballot;
                const long long n0 = timeIt ? clock64() : 0;
                while(ballot) {
                    const unsigned int b = __ffs(ballot) - 1u;
                    ballot &= ballot - 1u;
                    const unsigned int id = __shfl_sync(0xFFFFFFFFu, (unsigned int)myIndex, b);
                    if(space.shift != 0xFFFFFFFFu) {
                        const uint2 *row = space.rows + ((unsigned long long)(id - space.first_row) << space.shift);
                        if(SHARDED && L.world > 1) {
                            returned += nearDeliverRow<true>(row, space.shift, space.peer_shift, L.near_rings, L.num_rings, L.rank, k, state,
                                                             &outbox, (unsigned int)((done0 + step + 1) & 1ull));
                        }
                        else {
                            nearDeliverRow<false>(row, space.shift, space.peer_shift, L.near_rings, L.num_rings, 0u, k, state);
                        }
                    }
                }
                // additions into another GPU's rings must have landed there before that GPU is told (after
                // the barrier below) that this step is complete
                const long long n1 = timeIt ? clock64() : 0;
                // (with queues the thread that sends the header fences, and only if some entry went the direct way)
                if(SHARDED && !outbox.words && __any_sync(0xFFFFFFFFu, returned != 0.0f)) __threadfence_system();
                if(timeIt && lane == 0) {       // probes 8-10: near delivery, the fence behind it, spiking warps
                    atomicAdd(&state->probe[8], (unsigned long long)(n1 - n0));
                    atomicAdd(&state->probe[9], (unsigned long long)(clock64() - n1));
                    atomicAdd(&state->probe[10], 1ull);
                }
            }
        }
        // spike-queue update for the next step (neuronUpdateGroupMerged.cc:947-975)
        if(blockIdx.x == 0 && threadIdx.x < numGroups) {
            const b200_neuron_group &o = L.neuron.groups[threadIdx.x];
            o.spk_cnt[ringSlot(k + 2, o.num_delay_slots)] = 0;
        }
        if(prof) c3 = clock64();
        const bool queued = SHARDED && emit && L.world > 1 && outbox.words != 0u;
        if(queued && step + 1 < L.num_steps) {
            // Near synapses between processes.  Out: the header of this CTA's queue in every other process's
            // arena (the entries went out while the neurons were updated).  In: the queues the CTAs of this
            // index in the other processes filled for this process, added into its rings BEFORE this CTA
            // arrives at the barrier, so that the next neuron update finds them.  A queue of this step's
            // parity is written again two steps on: by then its sender has passed a barrier that every CTA of
            // this process reached only behind its own sends of the step in between, hence behind this read.
            // (Across launches: a launch starts by fetching every process's spike counts of the step before,
            // which those publish behind their last barrier.)
            const long long x0 = prof ? clock64() : 0;
            chainSync(chainThreads);
            const unsigned long long tag = done0 + step + 1;
            const unsigned long long parityWords = (tag & 1ull) * outbox.parity_words;
            if(threadIdx.x < L.world && threadIdx.x != L.rank) {
                if(outbox.fenced) __threadfence_system();
                const unsigned int n = min(outbox.count[threadIdx.x], outbox.words - 1u);
                storeRelaxedSys(outbox.queue[threadIdx.x] + parityWords, (tag << 32) | n);
                outbox.count[threadIdx.x] = 0u;
            }
            for(unsigned int p = warp; p < L.world; p += chainWarps) {
                if(p == L.rank) continue;
                unsigned long long *queue = reinterpret_cast<unsigned long long*>(L.arena + L.queue_offset) + parityWords +
                    ((unsigned long long)p * L.queue_count + blockIdx.x) * L.queue_words;
                unsigned int n = 0;
                if(lane == 0) {
                    const long long h0 = L.profile ? clock64() : 0;
                    n = min(awaitWord(queue, tag, state), outbox.words - 1u);
                    // probe 7: CTA 0's wait for the headers of the other processes (summed over them)
                    if(L.profile && blockIdx.x == 0) atomicAdd(&state->probe[7], (unsigned long long)(clock64() - h0));
                }
                n = __shfl_sync(0xFFFFFFFFu, n, 0);
                for(unsigned int i = lane; i < n; i += 32u) {
                    unsigned long long e = 0, polls = 0;
                    while((e = loadRelaxedSys(queue + 1u + i)) == 0ull) {
                        if(++polls > state->exchange_spin_limit) {
                            atomicOr(&state->error, ERR_EXCHANGE_TIMEOUT);
                            break;
                        }
                    }
                    if(e == 0ull) continue;
                    storeRelaxedSys(queue + 1u + i, 0ull);
                    const unsigned int word = (unsigned int)e;
                    const NearRing &ring = L.near_rings[L.rank * L.num_rings + ((word >> 1) & 0x7Fu)];
                    const unsigned int post = word >> 8;
                    if(post < ring.num_neurons) {
                        redAdd(ring.den_delay + (unsigned long long)ringSlot(k + 2u + (word & 1u), ring.D) * ring.num_neurons + post,
                               __uint_as_float((unsigned int)(e >> 32)));
                    }
                    else {
                        atomicOr(&state->error, ERR_IND_RANGE);
                    }
                }
            }
            if(prof) sh.waited[1] += (unsigned long long)(clock64() - x0);
        }
        if(emit && threadIdx.x == 0 && step >= 2) {
            // the stream warps that took pass step-1 (the spikes of the step before last; this CTA's
            // if the parities match) must be through it: the barrier below is the last one ahead of
            // the first neuron update that may read what they delivered
            const long long since = clock64();
            for(unsigned int w = 0; w < streamWarps && (gridDim.x < 2u || ((step - 1) & 1u) == (blockIdx.x & 1u)); w++) {
                while(sh.streamDone[w] < (unsigned int)(step - 1)) {
                    if(clock64() - since > state->stream_wait_cycles) {
                        atomicOr(&state->error, ERR_BARRIER_TIMEOUT);
                        break;
                    }
                }
            }
            // (no fence of its own: the release at the barrier below follows in program order and is
            // cumulative over what this thread has just observed)
            if(prof) cyc[5] += (unsigned long long)(clock64() - since);
        }
        const long long a0 = prof ? clock64() : 0;
        arrive();
        // probe 11: CTA 0's arrival (its warps' waits for the other processes' queues end here)
        if(prof && blockIdx.x == 0) atomicAdd(&state->probe[11], (unsigned long long)(clock64() - a0));
        // (emit schedule, per CTA, in the slot the other schedules use for the header wait: from the start of the
        // step to this CTA's arrival)
        if(prof && emit) cyc[4] += (unsigned long long)(clock64() - c0);
        if(queued && threadIdx.x == 0) outbox.fenced = 0u;
        // every chain thread is past its neuron update: the tag of the NEXT step's spike words may change
        if(SHARDED && emit && L.world > 1 && threadIdx.x == 0) exchange.tag = done0 + step + 2;
        if(emit && mine && myActive && step + 1 < L.num_steps) {
            drawCurrentSources<NCS>(L.neuron, L.neuron.groups[myGroup], 0u, (unsigned int)myIndex, t0 + step + 1, csCount);
        }
        // (sharded model without a publisher warp: the chain's last warp of CTA 0 tells every process how many
        // spikes each population emitted)
        if(SHARDED && L.world > 1 && !publisherWarps && blockIdx.x == 0 && warp == chainWarps - 1u) {
            if(lane == 0) {
                unsigned long long polls = 0;
                while(loadAcquire(L.barrier) < epoch) {
                    if(++polls > state->barrier_spin_limit) {
                        atomicOr(&state->error, ERR_BARRIER_TIMEOUT);
                        break;
                    }
                }
            }
            __syncwarp();
            for(unsigned int idx = lane; idx < L.world * numGroups; idx += 32u) {
                const unsigned int peer = idx / numGroups, gi = idx - peer * numGroups;
                const b200_neuron_group &g = L.neuron.groups[gi];
                const unsigned int wslot = ringSlot(k + 1u, g.num_delay_slots);
                const unsigned long long tag = ((done0 + step + 1) << 32) | (unsigned long long)__ldcg(&g.spk_cnt[wslot]);
                unsigned long long *cell = reinterpret_cast<unsigned long long*>(&g.spk_tag[wslot]);
                if(peer != L.rank) {
                    cell = reinterpret_cast<unsigned long long*>(peerArena[peer] + (reinterpret_cast<unsigned char*>(cell) - L.arena));
                }
                storeRelaxedSys(cell, tag);
            }
        }
        // emit mode of a sharded model: the next neuron update reads what the other processes' spiking
        // threads pushed into this process's rings, so their step must be complete too
        // (with queues, the headers this CTA has waited for above say the same of the CTAs that can reach it)
        if(!((SHARDED && emit && L.world > 1 && !queued) ? wait(done0 + step + 1, ringSlot(k + 1u, L.neuron.groups[0].num_delay_slots)) : wait())) B200_CHAIN_ABORT();
        if(emit && threadIdx.x == 0) sh.stepPassed = (unsigned int)(step + 1);    // the stream may read this step's spikes
        k = (k + 1 == period) ? 0u : k + 1;
        if(prof) {
            const long long c4 = clock64();
            cyc[0] += (unsigned long long)(c1 - c0);
            cyc[1] += (unsigned long long)(c2 - c1);
            cyc[2] += (unsigned long long)(c3 - c2);
            cyc[3] += (unsigned long long)(c4 - c3);
        }
    }
    #undef B200_CHAIN_ABORT
    if(prof) {
        if(blockIdx.x == 0) {
            for(int i = 0; i < 4; i++) state->phase_cycles[i] += cyc[i];
            state->probe[2] += cyc[5];      // probe 2: chain waiting for the stream warps
            state->probe[5] += sh.waited[0];
            state->probe[6] += sh.waited[1];
        }
        if(L.cta_cycles) {
            for(int i = 0; i < 4; i++) L.cta_cycles[4ull * blockIdx.x + i] += cyc[i];
            L.cta_cycles[4ull * gridDim.x + blockIdx.x] += cyc[4];
        }
    }
    if(mine && myActive) storeNeuron(L.neuron.groups[myGroup], myIndex, regs, true);
    if(blockIdx.x == 0 && threadIdx.x == 0) {
        state->timestep = t0 + L.num_steps;
        state->steps_done = state->steps_done + L.num_steps;
        state->phase = k;
    }
}
}   // namespace b200
