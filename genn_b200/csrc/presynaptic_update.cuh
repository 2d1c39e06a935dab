// Presynaptic update kernels: propagate the spikes of the previous step
// through SPARSE, BITMASK and DENSE connectivity into the target's input
// buffer (outPost) or dendritic-delay ring (denDelay).  Replace the
// reference's updatePresynapticKernel and its PostSpan / PreSpan /
// PostSpanBitmask strategies (backendSIMT.cc:694-764,
// presynapticUpdateStrategySIMT.cc:57-745).
//
// SPARSE.  The reference gives each block `blockSize` columns of the ragged
// matrix and makes it walk EVERY spike with scalar 4-byte loads, so its
// parallel width is maxRowLength threads per group however many spikes there
// are.  Here the work item is (spike, 512-synapse tile of that spike's row):
// grid = (row tiles of all merged groups, spike lanes, batch); block (c, y)
// handles tile c of spikes y, y+Y, y+2Y...  Within a tile each thread owns FOUR
// consecutive synapses whose first index is a multiple of four counted from the
// array base, so weights come in as one 128-bit load, uint16 indices as one
// 64-bit load (uint32: 128-bit, uint8: 32-bit) and delays as one 32-bit load,
// whatever the row stride: rows are not aligned in the reference's layout
// (stride = maxRowLength), so the tile is aligned to the array instead and the
// head/tail lanes that fall outside the row are masked.  Every warp-level load
// is a run of whole 32-byte sectors.  The scatter is a fire-and-forget fp32
// reduction into L2-resident targets; lanes of a warp that hit the same address
// are merged first when the target population is small enough for that to be
// likely.
//
// Algorithmic HBM bytes per synaptic event: sizeof(ind) + 4 (weight) + 1
// (delay, if any): 7 for the Potjans microcircuit with uint16 indices.
#pragma once

#include "common.cuh"
#include "init.cuh"

namespace b200
{
constexpr int PRE_BLOCK = 128;
constexpr int PRE_VEC = 4;
constexpr int PRE_TILE = PRE_BLOCK * PRE_VEC;     // synapses per block per spike

struct SynapseLaunch
{
    const b200_synapse_group *groups;
    const unsigned int *block_start;
    unsigned int num_groups;
    unsigned int batch;
    float dt;
    unsigned long long seed;
    StepState *state;
    unsigned int count_events;
    const unsigned char *tiled_served;  // per SPARSE group: 1 if the target-tiled kernel delivers it in heavy steps; or NULL
};

template<typename T> struct IndLoad;
template<> struct IndLoad<uint8_t>
{
    static __device__ __forceinline__ void load4(const void *base, unsigned long long idx, unsigned int (&out)[4])
    {
        const unsigned int w = __ldg(reinterpret_cast<const unsigned int*>(static_cast<const uint8_t*>(base) + idx));
        out[0] = w & 0xFFu; out[1] = (w >> 8) & 0xFFu; out[2] = (w >> 16) & 0xFFu; out[3] = w >> 24;
    }
};
template<> struct IndLoad<uint16_t>
{
    static __device__ __forceinline__ void load4(const void *base, unsigned long long idx, unsigned int (&out)[4])
    {
        const uint2 w = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(base) + idx));
        out[0] = w.x & 0xFFFFu; out[1] = w.x >> 16; out[2] = w.y & 0xFFFFu; out[3] = w.y >> 16;
    }
};
template<> struct IndLoad<uint32_t>
{
    static __device__ __forceinline__ void load4(const void *base, unsigned long long idx, unsigned int (&out)[4])
    {
        const uint4 w = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint32_t*>(base) + idx));
        out[0] = w.x; out[1] = w.y; out[2] = w.z; out[3] = w.w;
    }
};

// One (spike, tile) work item of a SPARSE group with a non-learning weight
// update model.
// `quad` is this thread's position in the row counted in groups of four
// synapses from the row's aligned start.
template<typename IndT>
__device__ __forceinline__ void sparseQuad(const b200_synapse_group &g, unsigned int pre, unsigned int quad,
                                           float *__restrict__ target, unsigned int denFront,
                                           StepState *state, unsigned int zeroDelay = 0u)
{
    // The row length and the row data are fetched TOGETHER (one memory round
    // trip, not two): the quad's address does not depend on the length, and a
    // quad past the end of its row still lies inside the array (or its tail
    // padding), so the loads are safe and simply discarded.
    const unsigned long long rowStart = (unsigned long long)pre * g.row_stride;
    const unsigned long long idx = (rowStart & ~3ull) + (unsigned long long)quad * PRE_VEC;
    if(idx >= (unsigned long long)g.num_src * g.row_stride) return;
    const unsigned int len = __ldg(&g.row_length[pre]);
    unsigned int post[4];
    IndLoad<IndT>::load4(g.ind, idx, post);
    float w[4];
    if(g.wu_model == B200_WU_STATIC_PULSE_CONSTANT_WEIGHT) {
        w[0] = w[1] = w[2] = w[3] = g.wu_params[0];
    }
    else {
        const float4 wv = __ldg(reinterpret_cast<const float4*>(g.g + idx));
        w[0] = wv.x; w[1] = wv.y; w[2] = wv.z; w[3] = wv.w;
    }
    const unsigned int D = g.max_den_delay;
    unsigned int dw = 0;
    if(D) dw = __ldg(reinterpret_cast<const unsigned int*>(g.d + idx));
    const unsigned long long rowEnd = rowStart + len;
    if(idx >= rowEnd) return;
    const unsigned int numTrg = g.num_trg;

#pragma unroll
    for(int j = 0; j < PRE_VEC; j++) {
        const unsigned long long s = idx + j;
        if(s >= rowStart && s < rowEnd) {
            unsigned int p = post[j];
            if(p >= numTrg) {
                atomicOr(&state->error, ERR_IND_RANGE);
                continue;
            }
            if(D) {
                unsigned int slot = denFront + ((dw >> (8 * j)) & 0xFFu);
                while(slot >= D) slot -= D;         // a delay of the ring length or more wraps around
                // zeroDelay says what to do with a synapse that arrives in the same step (its
                // slot is the front one): 0 deliver it, 1 the caller relies on there being
                // none, 2 somebody else delivers it, 3 somebody else delivers it and those
                // that arrive one step later
                if(zeroDelay) {
                    if(slot == denFront) {
                        if(zeroDelay == 1u) atomicOr(&state->error, ERR_DELAY_RANGE);
                        continue;
                    }
                    if(zeroDelay == 3u && slot == ((denFront + 1u == D) ? 0u : denFront + 1u)) continue;
                }
                redAdd(target + (unsigned long long)slot * numTrg + p, w[j]);
            }
            else {
                redAdd(target + p, w[j]);
            }
        }
    }
}

// SPARSE with a learning rule: the pre-spike half of STDP reads and writes the
// per-batch weight (weightUpdateModels.h:354-361).  Scalar per-synapse path.
template<typename IndT>
__device__ __forceinline__ void sparseTileSTDP(const b200_synapse_group &g, unsigned int pre, unsigned int tile,
                                               unsigned int b, float t, unsigned int k)
{
    const unsigned int len = __ldg(&g.row_length[pre]);
    const unsigned long long rowStart = (unsigned long long)pre * g.row_stride;
    const unsigned long long perBatch = (unsigned long long)g.num_src * g.row_stride;
    float *gb = g.g + (unsigned long long)b * perBatch;
    const unsigned int tslots = g.trg_delay_slots;
    const float *stPost = g.trg_spike_times +
        ((unsigned long long)b * tslots + ringSlot(k + tslots - g.back_prop_delay, tslots)) * g.num_trg;
    float *out = g.out_post + (unsigned long long)b * g.num_trg;
#pragma unroll
    for(int j = 0; j < PRE_VEC; j++) {
        const unsigned int col = tile * PRE_TILE + j * PRE_BLOCK + threadIdx.x;
        if(col < len) {
            const unsigned long long s = rowStart + col;
            const unsigned int p = static_cast<const IndT*>(g.ind)[s];
            const float w = gb[s];
            redAdd(out + p, w);
            const float dts = B200_FSUB(t, B200_FADD(g.wu_params[7], stPost[p]));
            if(dts > 0.0f) {
                const float timing = expf(B200_FDIV(-dts, g.wu_params[1]));
                const float nw = B200_FSUB(w, B200_FMUL(g.wu_params[3], timing));
                gb[s] = fmaxf(g.wu_params[4], fminf(g.wu_params[5], nw));
            }
        }
    }
}

// One launch for every SPARSE merged group.
__global__ void __launch_bounds__(PRE_BLOCK)
presynapticSparseKernel(const SynapseLaunch L)
{
    const unsigned int gi = findGroup(L.block_start, L.num_groups, blockIdx.x);
    const b200_synapse_group &g = L.groups[gi];
    const unsigned int tile = blockIdx.x - __ldg(&L.block_start[gi]);
    const unsigned int b = blockIdx.z;
    if(L.tiled_served && L.tiled_served[gi] && L.state->heavy) return;
    const unsigned int k = L.state->phase;
    const unsigned int slots = g.src_delay_slots;
    const unsigned int rslot = ringSlot(k + slots - g.axonal_delay, slots);
    const unsigned int count = g.src_spk_cnt[b * slots + rslot];
    if(blockIdx.y >= count) return;
    const unsigned int *spk = g.src_spk + ((unsigned long long)b * slots + rslot) * g.num_src;
    const unsigned int D = g.max_den_delay;
    const unsigned int denFront = D ? ringSlot(k + 1, D) : 0;
    float *target = D ? g.den_delay + (unsigned long long)b * D * g.num_trg
                      : g.out_post + (unsigned long long)b * g.num_trg;
    const bool learn = (g.wu_model == B200_WU_STDP);
    const float t = B200_FMUL((float)L.state->timestep, L.dt);

    for(unsigned int s = blockIdx.y; s < count; s += gridDim.y) {
        const unsigned int pre = spk[s];
        if(learn) {
            switch(g.ind_bytes) {
            case 1: sparseTileSTDP<uint8_t>(g, pre, tile, b, t, k); break;
            case 2: sparseTileSTDP<uint16_t>(g, pre, tile, b, t, k); break;
            default: sparseTileSTDP<uint32_t>(g, pre, tile, b, t, k); break;
            }
        }
        else {
            switch(g.ind_bytes) {
            case 1: sparseQuad<uint8_t>(g, pre, tile * PRE_BLOCK + threadIdx.x, target, denFront, L.state); break;
            case 2: sparseQuad<uint16_t>(g, pre, tile * PRE_BLOCK + threadIdx.x, target, denFront, L.state); break;
            default: sparseQuad<uint32_t>(g, pre, tile * PRE_BLOCK + threadIdx.x, target, denFront, L.state); break;
            }
        }
        if(L.count_events && tile == 0 && threadIdx.x == 0) {
            atomicAdd(&L.state->synaptic_events, (unsigned long long)__ldg(&g.row_length[pre]));
        }
    }
}

// BITMASK and DENSE: one thread per postsynaptic neuron accumulates over the
// whole spike list in a register and issues a single reduction at the end
// (presynapticUpdateStrategySIMT.cc:295-306, 352-370).  BITMASK rows are padded
// to 32 so the 32 lanes of a warp test bits of ONE connectivity word, fetched
// with a single broadcast load: numPost/8 bytes per spike.  DENSE streams one
// coalesced weight row per spike: 4*numPost bytes per spike.
__global__ void __launch_bounds__(PRE_BLOCK)
presynapticPostSpanKernel(const SynapseLaunch L)
{
    const unsigned int gi = findGroup(L.block_start, L.num_groups, blockIdx.x);
    const b200_synapse_group &g = L.groups[gi];
    const unsigned int post = (blockIdx.x - __ldg(&L.block_start[gi])) * PRE_BLOCK + threadIdx.x;
    const unsigned int b = blockIdx.z;
    const unsigned int k = L.state->phase;
    const unsigned int slots = g.src_delay_slots;
    const unsigned int rslot = ringSlot(k + slots - g.axonal_delay, slots);
    const unsigned int count = g.src_spk_cnt[b * slots + rslot];
    if(count == 0 || post >= g.row_stride) return;
    const unsigned int *spk = g.src_spk + ((unsigned long long)b * slots + rslot) * g.num_src;
    const unsigned int numTrg = g.num_trg;
    const bool valid = post < numTrg;
    float acc = 0.0f;
    unsigned int events = 0;

    if(g.connectivity == B200_CONN_BITMASK) {
        const float w = g.wu_params[0];
        const unsigned int bit = 0x80000000u >> (post & 31u);
        for(unsigned int s = 0; s < count; s++) {
            const unsigned long long gid = (unsigned long long)spk[s] * g.row_stride + post;
            if(__ldg(&g.gp[gid >> 5]) & bit) {
                acc = B200_FADD(acc, w);
                events++;
            }
        }
    }
    else if(g.wu_model == B200_WU_STDP) {
        if(!valid) return;
        const float t = B200_FMUL((float)L.state->timestep, L.dt);
        const unsigned int tslots = g.trg_delay_slots;
        const float stPost = g.trg_spike_times[((unsigned long long)b * tslots +
                                                ringSlot(k + tslots - g.back_prop_delay, tslots)) * numTrg + post];
        float *gb = g.g + (unsigned long long)b * g.num_src * numTrg;
        const float dts = B200_FSUB(t, B200_FADD(g.wu_params[7], stPost));
        for(unsigned int s = 0; s < count; s++) {
            const unsigned long long id = (unsigned long long)spk[s] * numTrg + post;
            const float w = gb[id];
            acc = B200_FADD(acc, w);
            if(dts > 0.0f) {
                const float timing = expf(B200_FDIV(-dts, g.wu_params[1]));
                const float nw = B200_FSUB(w, B200_FMUL(g.wu_params[3], timing));
                gb[id] = fmaxf(g.wu_params[4], fminf(g.wu_params[5], nw));
            }
        }
        events = count;
    }
    else {
        if(!valid) return;
        const bool constant = (g.wu_model == B200_WU_STATIC_PULSE_CONSTANT_WEIGHT);
        for(unsigned int s = 0; s < count; s++) {
            const float w = constant ? g.wu_params[0] : __ldg(&g.g[(unsigned long long)spk[s] * numTrg + post]);
            acc = B200_FADD(acc, w);
        }
        events = count;
    }
    if(valid && events) redAdd(g.out_post + (unsigned long long)b * numTrg + post, acc);
    if(L.count_events && events) atomicAdd(&L.state->synaptic_events, (unsigned long long)events);
}

// PROCEDURAL connectivity (presynapticUpdateStrategySIMT.cc:394-566): nothing of the matrix is
// stored; the row of every spiking neuron is regenerated from its Philox streams, exactly as the
// initialisation kernel would have written it (generateRow, init.cuh), and so is every weight that
// is not a constant (the stream of a weight is keyed on pre * row_stride + position in the row, as in
// initSparseVarKernel).
//
// A work item is (spike, sub-row): T = connectSubRows() threads share one row, each regenerating the
// synapses onto its own range of targets from its own stream (T a power of two of at most 32, so the
// T items of a spike are neighbouring lanes of one warp).  The items of a (group, batch entry) are
// spread over the whole grid: grid (x, groups, batch) with a grid-stride loop over the items, since
// the number of spikes is only known on the device.  Every synapse costs one reduction into L2 and
// no HBM traffic at all.
constexpr unsigned int PROC_BLOCK = 256;
constexpr unsigned int PROC_HOLD = 48;      // targets of a sub-row kept between its generation and its delivery

__global__ void __launch_bounds__(PROC_BLOCK)
presynapticProceduralKernel(const SynapseLaunch L)
{
    const b200_synapse_group &g = L.groups[blockIdx.y];
    const unsigned int b = blockIdx.z;
    const unsigned int lane = threadIdx.x & 31u;
    const unsigned int k = L.state->phase;
    const unsigned int slots = g.src_delay_slots;
    const unsigned int rslot = ringSlot(k + slots - g.axonal_delay, slots);
    const unsigned int count = g.src_spk_cnt[b * slots + rslot];
    const unsigned int *spk = g.src_spk + ((unsigned long long)b * slots + rslot) * g.num_src;
    const unsigned int numTrg = g.num_trg;
    const unsigned int D = g.max_den_delay;
    // dendritic delay is not generated procedurally: slot 0 of a ring is the front
    float *target = (D ? g.den_delay + ((unsigned long long)b * D + ringSlot(k + 1, D)) * numTrg : g.out_post + (unsigned long long)b * numTrg);
    const bool constant = (g.wu_model == B200_WU_STATIC_PULSE_CONSTANT_WEIGHT);
    const unsigned int T = connectSubRows(g.proc_connect, g.proc_connect_params);
    const unsigned long long items = (unsigned long long)count * T;
    // whole warps stay in the loop together: the sub-rows of a spike exchange their lengths by shuffle
    const unsigned long long itemsPadded = (items + 31ull) & ~31ull;
    for(unsigned long long item = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; item < itemsPadded;
        item += (unsigned long long)gridDim.x * blockDim.x) {
        const bool live = item < items;
        const unsigned int s = (unsigned int)(item / T), t = (unsigned int)(item - (unsigned long long)s * T);
        unsigned int pre = live ? spk[s] : 0u;
        if(live && pre >= g.num_src) {
            atomicOr(&L.state->error, ERR_IND_RANGE);
            pre = 0xFFFFFFFFu;
        }
        const bool work = live && pre != 0xFFFFFFFFu;
        const unsigned int fixedLength = !work ? 0u : (g.proc_connect == B200_CONNECT_FIXED_NUMBER_POST_WITH_REPLACEMENT)
            ? (unsigned int)g.proc_connect_params[0] : (g.row_length ? g.row_length[pre] : 0u);
        auto deliver = [&](unsigned int at, unsigned int post) {
            if(at >= g.row_stride) return;      // the row the initialisation kernel would have stored ends here
            float w = g.wu_params[0];
            if(!constant) {
                b200_rng rng = b200_rng_init(L.seed, g.proc_weight_stream, (unsigned long long)pre * g.row_stride + at);
                w = drawInitValue(g.proc_weight_init, g.proc_weight_params, &rng);
            }
            redAdd(target + post, w);
        };
        unsigned int n = 0;
        if(!constant && T > 1u) {
            // Drawn weights are keyed on the position in the ROW, which a sub-row only knows once the sub-rows
            // before it have been counted: generate the sub-row once into a small buffer, exchange the counts
            // (shuffle scan over the T lanes of the spike), then draw the weights and deliver from the buffer.
            // (A sub-row longer than the buffer is generated a second time for its tail.)
            unsigned int held[PROC_HOLD];
            if(work) n = generateRow(g.proc_connect, g.proc_connect_params, pre, 0u, numTrg, fixedLength, L.seed, g.rng_stream,
                                     [&](unsigned int at, unsigned int post) { if(at < PROC_HOLD) held[at] = post; }, t, t + 1u);
            unsigned int incl = n;
            for(unsigned int o = 1; o < T; o <<= 1) {
                const unsigned int v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if((lane & (T - 1u)) >= o) incl += v;
            }
            const unsigned int base = incl - n;
            const unsigned int fromBuffer = min(n, PROC_HOLD);
            for(unsigned int at = 0; at < fromBuffer; at++) deliver(base + at, held[at]);
            if(n > PROC_HOLD) {
                generateRow(g.proc_connect, g.proc_connect_params, pre, 0u, numTrg, fixedLength, L.seed, g.rng_stream,
                            [&](unsigned int at, unsigned int post) { if(at >= PROC_HOLD) deliver(base + at, post); }, t, t + 1u);
            }
        }
        else if(work) {
            n = generateRow(g.proc_connect, g.proc_connect_params, pre, 0u, numTrg, fixedLength, L.seed, g.rng_stream, deliver, t, t + 1u);
        }
        // the whole row's length: sum over the T lanes of the spike
        unsigned int rowLen = n;
        for(unsigned int o = 1; o < T; o <<= 1) rowLen += __shfl_xor_sync(0xFFFFFFFFu, rowLen, o);
        if(work && t == 0u) {
            if(rowLen > g.row_stride) atomicOr(&L.state->error, ERR_IND_RANGE);
            if(L.count_events) atomicAdd(&L.state->synaptic_events, (unsigned long long)min(rowLen, g.row_stride));
        }
    }
}
}   // namespace b200
