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

namespace b200
{
// Backstop for the waits between the two sets of warps (clock cycles, about half a minute): every
// wait of the other side is itself bounded and far shorter, so this only ends a CTA whose partner died.
constexpr long long STREAM_WAIT_CYCLES = 1ll << 36;

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
    bool barrierOk;
};

// One pass over one of the two item lists of every source, for the spikes whose
// header sits in buffer `buf`: warp `first` of `stride` takes every stride-th item.
__device__ __forceinline__ void deliverItems(const FusedLaunch &L, const StreamShared &sh, unsigned int buf,
                                             bool urgentList, unsigned int first, unsigned int stride,
                                             unsigned int k, unsigned long long stepsDone, StepState *state)
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
                    const unsigned int zeroDelay = urgentList ? 0u : (L.urgent && L.urgent[item.x].stride) ? 2u : 1u;
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

template<int NPSM, int NCS>
__global__ void __launch_bounds__(FUSED_BLOCK, 1)
streamStepKernel(FusedLaunch L)
{
    extern __shared__ __align__(16) unsigned char fusedSmem[];
    __shared__ StreamShared sh;
    __shared__ unsigned char *peerArena[B200_MAX_RANKS];
    __shared__ ExchangeCtx exchange;
    if(threadIdx.x < B200_MAX_RANKS) peerArena[threadIdx.x] = L.peer_table ? L.peer_table[threadIdx.x] : nullptr;
    if(threadIdx.x < 32) sh.streamDone[threadIdx.x] = 0u;
    if(threadIdx.x == 0) {
        exchange.world = L.world;
        exchange.rank = L.rank;
        exchange.arena = L.arena;
        exchange.peers = peerArena;
        sh.headReady = 0u;
        sh.stop = 0u;
    }
    const ExchangeCtx *xp = (L.world > 1) ? &exchange : nullptr;
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
        }
    }
    __syncthreads();        // the last barrier every warp of the CTA takes part in

    const unsigned int lane = threadIdx.x & 31u;
    const unsigned int warp = threadIdx.x >> 5;
    const unsigned int warpsPerBlock = blockDim.x >> 5;
    const unsigned int streamWarps = L.stream_warps;
    const unsigned int chainWarps = warpsPerBlock - streamWarps;
    const unsigned int chainThreads = chainWarps * 32u;
    StepState *state = L.neuron.state;
    const unsigned int period = state->ring_period;
    unsigned int k = state->phase;
    const unsigned long long t0 = state->timestep;
    const unsigned long long done0 = state->steps_done;

    // =========================== stream warps ==================================================
    if(warp >= chainWarps) {
        const unsigned int me = warp - chainWarps;
        const unsigned int first = me * gridDim.x + blockIdx.x, stride = streamWarps * gridDim.x;
        unsigned long long busy = 0, idle = 0;
        for(unsigned long long step = 0; step < L.num_steps; step++) {
            const long long since = clock64();
            while(sh.headReady < (unsigned int)(step + 1)) {
                if(sh.stop) return;
                if(clock64() - since > STREAM_WAIT_CYCLES) {
                    if(lane == 0) atomicOr(&state->error, ERR_BARRIER_TIMEOUT);
                    return;
                }
                __nanosleep(40);
            }
            __threadfence_block();
            __syncwarp();
            const long long began = clock64();
            deliverItems(L, sh, (unsigned int)(step & 1u), false, first, stride, k, done0 + step, state);
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

    auto arrive = [&]() {
        chainSync(chainThreads);
        if(threadIdx.x == 0) {
            asm volatile("red.release.gpu.global.add.u64 [%0], %1;" :: "l"(L.barrier), "l"(1ull) : "memory");
        }
        epoch += gridDim.x;
    };
    auto wait = [&]() -> bool {
        if(threadIdx.x == 0) {
            unsigned long long polls = 0;
            bool good = true;
            while(loadAcquire(L.barrier) < epoch) {
                if(++polls > BARRIER_SPIN_LIMIT) {
                    atomicOr(&state->error, ERR_BARRIER_TIMEOUT);
                    good = false;
                    break;
                }
            }
            // one thread decides for all: a CTA whose chain threads disagreed would hang on its barrier
            if(__ldcg(&state->error) & (ERR_BARRIER_TIMEOUT | ERR_EXCHANGE_TIMEOUT)) good = false;
            sh.barrierOk = good;
        }
        chainSync(chainThreads);
        return sh.barrierOk;
    };

    const bool prof = L.profile && threadIdx.x == 0;
    long long c0 = 0, c1 = 0, c2 = 0, c3 = 0;
    unsigned long long cyc[6] = {0, 0, 0, 0, 0, 0};
    for(unsigned long long step = 0; step < L.num_steps; step++) {
        if(prof) c0 = clock64();
        const unsigned int buf = (unsigned int)(step & 1u);

        // ---------------- header: spike counts and first ids of every source ----------------------
        if(warp < (L.num_sources + 31u) / 32u) {
            const unsigned int si = warp * 32u + lane;
            unsigned int cnt = 0, rslot = 0;
            unsigned int ids[FUSED_PREFETCH_IDS];
            #pragma unroll
            for(unsigned int j = 0; j < FUSED_PREFETCH_IDS; j++) ids[j] = 0u;
            if(si < L.num_sources) {
                const FusedSource &src = L.sources[si];
                rslot = ringSlot(k + src.slots - src.delay, src.slots);
                if(src.spk_tag) {
                    // sharded model: (step, count) and (step, id) words written by the list's owner
                    // into THIS process's memory; poll (bounded) for the count of the step we need
                    const long long expected = (long long)(done0 + step) - (long long)src.delay;
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
        }
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
                    if(clock64() - since > STREAM_WAIT_CYCLES) {
                        atomicOr(&state->error, ERR_BARRIER_TIMEOUT);
                        break;
                    }
                }
            }
            __threadfence_block();
            if(prof) cyc[5] += (unsigned long long)(clock64() - since);
        }
        if(L.world > 1 && threadIdx.x == 0) exchange.tag = done0 + step + 1;    // read after the barrier below
        arrive();
        // in the shadow of the barrier: this step's random draws
        unsigned int csCount[NCS > 0 ? NCS : 1] = {0};
        if(mine && myActive) {
            drawCurrentSources<NCS>(L.neuron, L.neuron.groups[myGroup], 0u, (unsigned int)myIndex, t0 + step, csCount);
        }
        if(!wait()) B200_CHAIN_ABORT();
        if(prof) c2 = clock64();

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
            neuronEmit<true>(L.neuron, g, 0u, myLocal, spiked, k, t0 + step, t, xp);
        }
        // spike-queue update for the next step (neuronUpdateGroupMerged.cc:947-975)
        if(blockIdx.x == 0 && threadIdx.x < numGroups) {
            const b200_neuron_group &o = L.neuron.groups[threadIdx.x];
            o.spk_cnt[ringSlot(k + 2, o.num_delay_slots)] = 0;
        }
        if(prof) c3 = clock64();
        arrive();
        // sharded model: one warp waits for the last CTA and tells every process how many spikes
        // each population emitted ("step s: n spikes", one 64-bit store per process and population);
        // the ids already sit in every arena
        if(L.world > 1 && blockIdx.x == 0 && warp == chainWarps - 1u) {
            unsigned long long polls = 0;
            while(loadAcquire(L.barrier) < epoch) {
                if(++polls > BARRIER_SPIN_LIMIT) {
                    atomicOr(&state->error, ERR_BARRIER_TIMEOUT);
                    break;
                }
            }
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
        if(!wait()) B200_CHAIN_ABORT();
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
