// Target-stationary persistent time-step kernel ("owner" path).
//
// Every CTA OWNS a contiguous block of neurons for the whole launch: their
// state lives in registers and their dendritic-delay rings (or plain input
// accumulators) live in the CTA's shared memory.  Synaptic events are then
// shared-memory reductions done by the owner of the target, so
//   * no fp32 reduction ever goes to L2 (scattered global reductions retire at
//     about 1.9e11 sector operations per second on a B200, a third of what the
//     HBM stream of a 7-byte synapse could feed), and
//   * the presynaptic phase and the neuron phase of a step are separated by a
//     CTA barrier only.  The single GRID barrier left in a step is the spike
//     exchange: every CTA must know every spike of the step.
// The price is that each CTA reads only the part of a spike's row that targets
// its own neurons.  Rows sorted by postsynaptic index (the reference's own
// connectivity builders emit them sorted, and set_sparse_connections sorts) make
// that part a contiguous segment; a table of segment offsets per (row, owner) is
// built once at initialisation.  Models whose rows are not sorted, whose rings do
// not fit shared memory, or that learn, use the other paths.
//
// Measured on the Potjans microcircuit (B200): 10.5 us per step against 8.4 us for
// the kernel with global reductions.  Splitting ~180 spiking rows per step over
// ~40 owners each turns them into ~7 000 segments of about four synapses, i.e.
// ~29 000 scattered 32-byte DRAM reads per step instead of ~700 opened rows, and
// HBM retires random sectors at only a few 1e9 per second.  The path is therefore
// opt-in (option use_owner); it wins where rows are long relative to the number of
// owners.
//
// The reference has no counterpart: its presynaptic kernels scatter with global
// atomics from wherever the spike is processed
// (presynapticUpdateStrategySIMT.cc:295-316) and its kernels are separated by
// launches (backendCUDAHIP.cc:386-420, 548-589).
#pragma once

#include "common.cuh"
#include "neuron_update.cuh"
#include "fused_step.cuh"

namespace b200
{
constexpr int OWNER_BLOCK = 768;                 // one CTA per SM; also the most neurons a CTA can own
constexpr unsigned int OWNER_MAX_PIECES = 4;     // populations a CTA's block of neurons may span
constexpr unsigned int ERR_ROWS_UNSORTED = 16u;
// A work item is one spike's segment for one owner: a handful of synapses (a row
// of ~500 split over ~40 owners), so eight lanes serve it and a warp works on
// four items at once.
// (item_lanes in the launch structure: 8, 16 or 32)

struct OwnerPiece
{
    unsigned int group;                  // neuron group index
    unsigned int lo;                     // first owned neuron, relative to the group's first_neuron
    unsigned int n;                      // owned neurons of this group
    unsigned int thread0;                // first thread of the CTA serving the piece (multiple of 32)
    unsigned int tile[B200_MAX_PSM];     // float offset of each fused PSM's tile in shared memory
};

struct OwnerEntry
{
    unsigned int source;                 // index into the spike sources
    unsigned int sgroup;                 // index into the SPARSE group table
    unsigned int piece;                  // which piece of this CTA the group targets
    unsigned int boundary;               // ordinal of that piece among the owners of the target group
    unsigned int psm;                    // which fused PSM of the target group
    unsigned int num_bounds;             // offsets per row of this group's table
    const unsigned int *offsets;         // [numSrc][num_bounds]: start of each owner's segment in the row
};

struct OwnerCta
{
    unsigned int num_pieces;
    unsigned int num_entries;
    unsigned int entry_begin;
    unsigned int tile_floats;
    OwnerPiece piece[OWNER_MAX_PIECES];
};

struct OwnerLaunch
{
    NeuronLaunch neuron;
    const b200_synapse_group *sgroups;
    const FusedSource *sources;
    const OwnerCta *ctas;
    const OwnerEntry *entries;
    unsigned int num_sources;
    unsigned int num_sgroups;
    unsigned int table_bytes;            // shared memory reserved for the staged tables
    unsigned int item_lanes;             // lanes serving one work item: 8, 16 or 32
    unsigned int count_events;
    unsigned int profile;
    unsigned long long num_steps;
    unsigned long long *barrier;
    unsigned long long *cta_cycles;
};

// ---- initialisation: segment offsets and the sortedness check ------------------
template<typename IndT>
__global__ void __launch_bounds__(256)
ownerCheckSortedKernel(const unsigned int *__restrict__ row_length, const void *__restrict__ ind,
                       unsigned int num_src, unsigned int num_trg, unsigned int row_stride, StepState *state)
{
    const unsigned long long total = (unsigned long long)num_src * row_stride;
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for(unsigned long long e = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const unsigned int pre = (unsigned int)(e / row_stride);
        const unsigned int j = (unsigned int)(e - (unsigned long long)pre * row_stride);
        const unsigned int len = __ldg(&row_length[pre]);
        if(j < len) {
            const unsigned int a = static_cast<const IndT*>(ind)[e];
            if(a >= num_trg) atomicOr(&state->error, ERR_IND_RANGE);
            if(j + 1 < len && a > static_cast<const IndT*>(ind)[e + 1]) atomicOr(&state->error, ERR_ROWS_UNSORTED);
        }
    }
}

// offsets[row][j] = first position in the row whose postsynaptic index is >= bounds[j]
template<typename IndT>
__global__ void __launch_bounds__(256)
ownerBuildOffsetsKernel(const unsigned int *__restrict__ row_length, const void *__restrict__ ind,
                        unsigned int num_src, unsigned int row_stride, const unsigned int *__restrict__ bounds,
                        unsigned int num_bounds, unsigned int *offsets)
{
    const unsigned long long total = (unsigned long long)num_src * num_bounds;
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for(unsigned long long e = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const unsigned int pre = (unsigned int)(e / num_bounds);
        const unsigned int j = (unsigned int)(e - (unsigned long long)pre * num_bounds);
        const unsigned int target = __ldg(&bounds[j]);
        const IndT *row = static_cast<const IndT*>(ind) + (unsigned long long)pre * row_stride;
        unsigned int lo = 0, hi = __ldg(&row_length[pre]);
        while(lo < hi) {
            const unsigned int mid = (lo + hi) >> 1;
            if(row[mid] < target) lo = mid + 1; else hi = mid;
        }
        offsets[e] = lo;
    }
}

// ---- the kernel -----------------------------------------------------------------
template<typename IndT>
__device__ __forceinline__ void ownerSegment(const b200_synapse_group &g, unsigned long long base, unsigned int lo,
                                             unsigned int hi, float *tile, unsigned int n, unsigned int front,
                                             unsigned int firstPost, unsigned int lane, unsigned int lanes)
{
    const unsigned int D = g.max_den_delay;
    const bool constant = (g.wu_model == B200_WU_STATIC_PULSE_CONSTANT_WEIGHT);
    for(unsigned int k = lo + lane; k < hi; k += lanes) {
        const unsigned long long s = base + k;
        const unsigned int post = static_cast<const IndT*>(g.ind)[s] - firstPost;
        const float w = constant ? g.wu_params[0] : __ldg(&g.g[s]);
        unsigned int slot = 0;
        if(D) {
            slot = front + __ldg(&g.d[s]);
            while(slot >= D) slot -= D;
        }
        if(post < n) atomicAdd(&tile[slot * n + post], w);
    }
}

template<int NPSM, int NCS>
__global__ void __launch_bounds__(OWNER_BLOCK, 1)
ownerStepKernel(OwnerLaunch L)
{
    extern __shared__ __align__(16) unsigned char ownerSmem[];
    __shared__ bool barrierOk;
    __shared__ unsigned int headCnt[32], headSlot[32], headIds[32][FUSED_PREFETCH_IDS];
    __shared__ OwnerCta me;

    // ---- stage tables ---------------------------------------------------------------
    stageWords(&me, &L.ctas[blockIdx.x], sizeof(OwnerCta));
    unsigned char *p = ownerSmem;
    {
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
    }
    __syncthreads();
    const OwnerEntry *entries = reinterpret_cast<const OwnerEntry*>(p);
    stageWords(p, &L.entries[me.entry_begin], sizeof(OwnerEntry) * me.num_entries);
    float *tiles = reinterpret_cast<float*>(ownerSmem + L.table_bytes);

    const unsigned int lane = threadIdx.x & 31u;
    const unsigned int warp = threadIdx.x >> 5;
    const unsigned int numWarps = blockDim.x >> 5;
    StepState *state = L.neuron.state;
    const unsigned int period = state->ring_period;
    unsigned int k = state->phase;
    const unsigned long long t0 = state->timestep;
    unsigned long long epoch = 0;

    // ---- rings and accumulators of the owned neurons: global -> shared ----------------
    for(unsigned int q = 0; q < me.num_pieces; q++) {
        const OwnerPiece &pc = me.piece[q];
        const b200_neuron_group &g = L.neuron.groups[pc.group];
        for(unsigned int m = 0; m < g.num_psm; m++) {
            const unsigned int D = g.psm[m].max_den_delay;
            float *tile = tiles + pc.tile[m];
            const unsigned int rows = D ? D : 1u;
            for(unsigned int e = threadIdx.x; e < rows * pc.n; e += blockDim.x) {
                const unsigned int slot = e / pc.n, i = e - slot * pc.n;
                tile[e] = D ? __ldcg(&g.psm[m].den_delay[(unsigned long long)slot * g.num_neurons + g.first_neuron + pc.lo + i])
                            : 0.0f;
            }
        }
    }

    // ---- this thread's neuron -----------------------------------------------------------
    unsigned int myPiece = 0;
    bool mine = false;
    for(unsigned int q = 0; q < me.num_pieces; q++) {
        const unsigned int span = (me.piece[q].n + 31u) & ~31u;
        if(threadIdx.x >= me.piece[q].thread0 && threadIdx.x < me.piece[q].thread0 + span) {
            myPiece = q;
            mine = true;
        }
    }
    const OwnerPiece &pc = me.piece[myPiece];
    const unsigned int myOff = mine ? threadIdx.x - pc.thread0 : 0u;           // index inside the piece
    const b200_neuron_group &myG = L.neuron.groups[mine ? pc.group : 0u];
    const unsigned int myLocal = pc.lo + myOff;                                 // relative to first_neuron
    const bool myActive = mine && myOff < pc.n;
    const unsigned long long myIndex = myG.first_neuron + myLocal;
    NeuronRegs<NPSM, NCS> regs;
    if(myActive) loadNeuron<true>(myG, myIndex, regs);
    unsigned int csCount[NCS > 0 ? NCS : 1] = {0};
    if(myActive) drawCurrentSources<NCS>(L.neuron, myG, 0u, (unsigned int)myIndex, t0, csCount);
    __syncthreads();

    const bool prof = L.profile && threadIdx.x == 0;
    long long c0 = 0, c1 = 0, c2 = 0, c3 = 0;
    for(unsigned long long step = 0; step < L.num_steps; step++) {
        if(prof) c0 = clock64();
        // ---------------- spike header: counts and first ids of every source ---------------
        if(threadIdx.x < 32u) {
            unsigned int cnt = 0, rslot = 0;
            if(lane < L.num_sources) {
                const FusedSource &src = L.sources[lane];
                rslot = ringSlot(k + src.slots - src.delay, src.slots);
                const unsigned int *list = src.spk + (unsigned long long)rslot * src.num_src;
                unsigned int ids[FUSED_PREFETCH_IDS];
                cnt = __ldcg(&src.spk_cnt[rslot]);
                #pragma unroll
                for(unsigned int j = 0; j < FUSED_PREFETCH_IDS; j++) ids[j] = (j < src.num_src) ? __ldcg(&list[j]) : 0u;
                #pragma unroll
                for(unsigned int j = 0; j < FUSED_PREFETCH_IDS; j++) headIds[lane][j] = ids[j];
            }
            headCnt[lane] = cnt;
            headSlot[lane] = rslot;
        }
        __syncthreads();

        // ---------------- presynaptic phase: my segments of every spiking row ---------------
        for(unsigned int base = 0; base < me.num_entries; base += 32u) {
            const unsigned int e = base + lane;
            const unsigned int cnt = (e < me.num_entries) ? headCnt[entries[e].source] : 0u;
            unsigned int incl = cnt;
            #pragma unroll
            for(int o = 1; o < 32; o <<= 1) {
                const unsigned int v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if(lane >= o) incl += v;
            }
            const unsigned int total = __shfl_sync(0xFFFFFFFFu, incl, 31);
            const unsigned int itemLanes = L.item_lanes, itemsPerWarp = 32u / itemLanes;
            const unsigned int sub = lane / itemLanes, sl = lane % itemLanes;
            for(unsigned int it0 = warp * itemsPerWarp; it0 < total; it0 += numWarps * itemsPerWarp) {
                // each group of eight lanes finds the entry and spike of its own item
                unsigned int owner = 0, s = 0;
                for(unsigned int q = 0; q < itemsPerWarp; q++) {
                    const unsigned int itq = it0 + q;
                    const unsigned int found = __ballot_sync(0xFFFFFFFFu, incl > itq);
                    const unsigned int o = found ? (unsigned int)__ffs(found) - 1u : 0u;
                    const unsigned int oIncl = __shfl_sync(0xFFFFFFFFu, incl, o);
                    const unsigned int oCnt = __shfl_sync(0xFFFFFFFFu, cnt, o);
                    if(sub == q) {
                        owner = o;
                        s = itq - (oIncl - oCnt);
                    }
                }
                if(it0 + sub >= total) continue;
                const OwnerEntry &en = entries[base + owner];
                const FusedSource &src = L.sources[en.source];
                const unsigned int pre = (s < FUSED_PREFETCH_IDS)
                    ? headIds[en.source][s]
                    : __ldcg(&src.spk[(unsigned long long)headSlot[en.source] * src.num_src + s]);
                const b200_synapse_group &g = L.sgroups[en.sgroup];
                if(pre >= g.num_src) {
                    if(sl == 0) atomicOr(&state->error, ERR_IND_RANGE);
                    continue;
                }
                const unsigned int *off = en.offsets + (unsigned long long)pre * en.num_bounds + en.boundary;
                const unsigned int lo = __ldg(&off[0]), hi = __ldg(&off[1]);
                const OwnerPiece &tp = me.piece[en.piece];
                const b200_neuron_group &tg = L.neuron.groups[tp.group];
                const unsigned int D = g.max_den_delay;
                float *tile = tiles + tp.tile[en.psm];
                const unsigned int front = D ? ringSlot(k + 1, D) : 0u;
                const unsigned long long rowBase = (unsigned long long)pre * g.row_stride;
                const unsigned int firstPost = tg.first_neuron + tp.lo;
                switch(g.ind_bytes) {
                case 1: ownerSegment<uint8_t>(g, rowBase, lo, hi, tile, tp.n, front, firstPost, sl, itemLanes); break;
                case 2: ownerSegment<uint16_t>(g, rowBase, lo, hi, tile, tp.n, front, firstPost, sl, itemLanes); break;
                default: ownerSegment<uint32_t>(g, rowBase, lo, hi, tile, tp.n, front, firstPost, sl, itemLanes); break;
                }
                if(L.count_events && sl == 0 && hi > lo) atomicAdd(&state->synaptic_events, (unsigned long long)(hi - lo));
            }
        }
        __syncthreads();
        if(prof) c1 = clock64();

        // ---------------- neuron phase ---------------------------------------------------------
        const unsigned long long timestep = t0 + step;
        const float t = B200_FMUL((float)timestep, L.neuron.dt);
        bool spiked = false;
        if(myActive) {
            float front[NPSM];
            #pragma unroll
            for(unsigned int m = 0; m < NPSM; m++) {
                front[m] = 0.0f;
                if(m < myG.num_psm) {
                    const unsigned int D = myG.psm[m].max_den_delay;
                    float *cell = tiles + pc.tile[m] + (D ? ringSlot(k + 1, D) : 0u) * pc.n + myOff;
                    const float v = *cell;
                    *cell = 0.0f;
                    if(D) front[m] = v; else regs.lin[m] = B200_FADD(regs.lin[m], v);
                }
            }
            spiked = neuronCompute(L.neuron, myG, 0u, (unsigned int)myIndex, timestep, t, regs, front, csCount);
        }
        if(mine) neuronEmit<true>(L.neuron, myG, 0u, myLocal, spiked, k, timestep, t);
        // spike-queue update for the next step (neuronUpdateGroupMerged.cc:947-975)
        if(blockIdx.x == 0 && threadIdx.x < L.neuron.num_groups) {
            const b200_neuron_group &o = L.neuron.groups[threadIdx.x];
            o.spk_cnt[ringSlot(k + 2, o.num_delay_slots)] = 0;
        }
        if(prof) c2 = clock64();

        // ---------------- the one grid barrier of the step: spike exchange ------------------------
        gridArrive(L.barrier, epoch);
        // in its shadow: the next step's random draws
        if(myActive) drawCurrentSources<NCS>(L.neuron, myG, 0u, (unsigned int)myIndex, timestep + 1, csCount);
        if(!gridWait(L.barrier, epoch, &barrierOk, state)) return;
        k = (k + 1 == period) ? 0u : k + 1;
        if(prof) {
            c3 = clock64();
            if(L.cta_cycles) {
                unsigned long long *m4 = L.cta_cycles + 4ull * blockIdx.x;
                m4[0] += (unsigned long long)(c1 - c0);
                m4[1] += 0ull;
                m4[2] += (unsigned long long)(c2 - c1);
                m4[3] += (unsigned long long)(c3 - c2);
            }
            if(blockIdx.x == 0) {
                state->phase_cycles[0] += (unsigned long long)(c1 - c0);
                state->phase_cycles[2] += (unsigned long long)(c2 - c1);
                state->phase_cycles[3] += (unsigned long long)(c3 - c2);
            }
        }
    }

    // ---- write everything the host may read back ---------------------------------------------
    __syncthreads();
    for(unsigned int q = 0; q < me.num_pieces; q++) {
        const OwnerPiece &wp = me.piece[q];
        const b200_neuron_group &g = L.neuron.groups[wp.group];
        for(unsigned int m = 0; m < g.num_psm; m++) {
            const unsigned int D = g.psm[m].max_den_delay;
            if(!D) continue;
            const float *tile = tiles + wp.tile[m];
            for(unsigned int e = threadIdx.x; e < D * wp.n; e += blockDim.x) {
                const unsigned int slot = e / wp.n, i = e - slot * wp.n;
                g.psm[m].den_delay[(unsigned long long)slot * g.num_neurons + g.first_neuron + wp.lo + i] = tile[e];
            }
        }
    }
    if(myActive) storeNeuron(myG, myIndex, regs, false);
    if(blockIdx.x == 0 && threadIdx.x == 0) {
        state->timestep = t0 + L.num_steps;
        state->steps_done = state->steps_done + L.num_steps;
        state->phase = k;
    }
}
}   // namespace b200
