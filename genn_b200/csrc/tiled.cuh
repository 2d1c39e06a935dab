// Target-tiled SPARSE delivery for steps with many spikes.
//
// One fp32 reduction into L2 per synaptic event (presynapticSparseKernel) tops out at the
// rate the L2 slices retire scattered reductions, far below HBM bandwidth.  Here the
// scatter is combined before it leaves the SM: the targets of every postsynaptic buffer
// (outPost, or a dendritic-delay ring) are cut into tiles whose accumulators
// [ring slot][target] fit one CTA's shared memory, events are added there with
// shared-memory atomics, and each touched cell is flushed to L2 once.
//
// That needs, for a spiking source neuron, its synapses into ONE tile as a contiguous run.
// The reference layout (rows per synapse group, presynapticUpdateStrategySIMT.cc:178-189)
// gives runs of two or three synapses per (row, tile) scattered over three arrays, so the
// library keeps a private re-packed copy of the non-learning SPARSE groups, rebuilt
// whenever the arrays it was made from change: per tile, the synapses of all groups onto
// that tile ordered by (group, source neuron), each as a key (delay << post_bits |
// target - first target of the tile; 16 bits when rings are at most 64 deep, else 32) and,
// unless every group has a constant weight, the fp32 weight; and per tile a table with the
// start of every source neuron's run.  A spike then costs one 8-byte table read and one
// contiguous run of about out-degree / tiles synapses per tile: 6 bytes per event with
// 16-bit keys against the 7 (uint16 indices) to 9 (uint32) of the reference layout.
//
// Work: 148 CTAs x 1024 threads, one per SM.  The (batch, tile, share of the spike list)
// items are dealt to the CTAs in contiguous, equally heavy stretches (weights: synapses per
// tile), so a CTA zeroes and flushes only one or two tiles.  Within an item a warp takes 32
// spikes at a time, reads their 32 run bounds, and walks the concatenation of the runs with
// all lanes busy (run found by a shuffle search over the prefix sums).
//
// A step with few events is cheaper on the one-reduction-per-event kernel (no tile to zero
// and flush); tiledDecideKernel estimates the step's events from the spike counts and both
// kernels obey its verdict.
#pragma once

#include "common.cuh"

namespace b200
{
constexpr int TILED_BLOCK = 1024;
constexpr unsigned int TILED_ACC_FLOATS = 45056;       // 176 KB of accumulators per CTA
constexpr unsigned int TILED_SPLIT = 8;                // shares of a spike list (items per tile and batch element)

struct TiledSource              // one non-learning SPARSE group, as a source of spikes for the tiles of its target
{
    const unsigned int *spk_cnt;
    const unsigned int *spk;
    unsigned int num_src;
    unsigned int src_delay_slots;
    unsigned int axonal_delay;
    unsigned int row_base;      // first row of the group in its target's tile tables
    float const_weight;
    float mean_row;             // synapses per source neuron (event estimate of a step)
};

struct TiledTile
{
    float *target;              // outPost [batch][N] or ring [batch][D][N]
    unsigned int num_trg;       // N
    unsigned int depth;         // D (1 for outPost)
    unsigned int first_trg;
    unsigned int num_tile;      // targets in this tile
    unsigned int stride;        // accumulator row stride (targets per tile of this buffer)
    unsigned int first_source, num_sources;     // into the TiledSource array
    unsigned int table;         // first entry of the tile's run-start table (rows of all its sources + 1)
};

struct TiledLaunch
{
    const TiledTile *tiles;
    const TiledSource *sources;
    const unsigned int *run_start;      // [entries]: absolute position of every (tile, row) run
    const void *keys;
    const float *weights;               // NULL: constant weights
    const unsigned int *cta_first_item; // [gridDim.x + 1]
    const unsigned short *item_tile;    // [items per batch element]
    const unsigned char *item_share;
    unsigned int items_per_batch;
    unsigned int num_sources;
    unsigned int batch;
    unsigned int post_bits;
    float min_events;
    StepState *state;
    unsigned int count_events;
};

// ---- building the private copy -----------------------------------------------------------------
struct TiledBuildGroup
{
    const unsigned int *row_length;
    const void *ind;
    const float *g;
    const unsigned char *d;
    unsigned int num_src, row_stride, ind_bytes, num_trg;
    unsigned int depth;             // ring depth of the target (1: outPost)
    unsigned int first_tile;        // first tile of the target buffer
    unsigned int stride;            // targets per tile
    unsigned int row_base;
    unsigned int rows_per_tile;     // table entries per tile of this target (rows of all its sources + 1)
    unsigned int first_table;       // table of the target's first tile
    float const_weight;
};

__device__ __forceinline__ unsigned int loadInd(const void *ind, unsigned int bytes, unsigned long long i)
{
    return (bytes == 1) ? static_cast<const uint8_t*>(ind)[i]
         : (bytes == 2) ? static_cast<const uint16_t*>(ind)[i] : static_cast<const uint32_t*>(ind)[i];
}

// pass 0: count the synapses of every (tile, row) run; pass 1: place them
template<typename KeyT>
__global__ void __launch_bounds__(256)
tiledBuildKernel(const TiledBuildGroup G, int pass, unsigned int *count, const unsigned int *run_start,
                 KeyT *keys, float *weights, unsigned int post_bits, StepState *state)
{
    const unsigned long long total = (unsigned long long)G.num_src * G.row_stride;
    const unsigned long long step = (unsigned long long)gridDim.x * blockDim.x;
    for(unsigned long long idx = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += step) {
        const unsigned int pre = (unsigned int)(idx / G.row_stride);
        const unsigned int j = (unsigned int)(idx - (unsigned long long)pre * G.row_stride);
        if(j >= G.row_length[pre]) continue;
        const unsigned int post = loadInd(G.ind, G.ind_bytes, idx);
        if(post >= G.num_trg) {
            atomicOr(&state->error, ERR_IND_RANGE);
            continue;
        }
        const unsigned int t = post / G.stride;
        const unsigned int entry = G.first_table + t * G.rows_per_tile + G.row_base + pre;
        if(pass == 0) {
            atomicAdd(&count[entry], 1u);
        }
        else {
            const unsigned int pos = run_start[entry] + atomicAdd(&count[entry], 1u);
            unsigned int delay = G.d ? G.d[idx] : 0u;
            delay %= G.depth;               // a delay of the ring length or more wraps around
            keys[pos] = (KeyT)((delay << post_bits) | (post - t * G.stride));
            if(weights) weights[pos] = G.g ? G.g[idx] : G.const_weight;
        }
    }
}

// ---- per step ----------------------------------------------------------------------------------
// Estimated synaptic events of the step from the spike counts; the verdict is read by the
// tiled kernel and by the one-reduction-per-event kernel.
__global__ void tiledDecideKernel(const TiledLaunch L)
{
    __shared__ float partial[32];
    const unsigned int k = L.state->phase;
    float est = 0.0f;
    for(unsigned int i = threadIdx.x; i < L.num_sources * L.batch; i += blockDim.x) {
        const TiledSource &s = L.sources[i / L.batch];
        const unsigned int b = i % L.batch;
        const unsigned int rslot = ringSlot(k + s.src_delay_slots - s.axonal_delay, s.src_delay_slots);
        est += (float)s.spk_cnt[b * s.src_delay_slots + rslot] * s.mean_row;
    }
    for(int o = 16; o > 0; o >>= 1) est += __shfl_xor_sync(0xFFFFFFFFu, est, o);
    if((threadIdx.x & 31u) == 0) partial[threadIdx.x >> 5] = est;
    __syncthreads();
    if(threadIdx.x == 0) {
        float sum = 0.0f;
        for(unsigned int w = 0; w < (blockDim.x + 31u) / 32u; w++) sum += partial[w];
        L.state->heavy = (sum >= L.min_events) ? 1u : 0u;
    }
}

__device__ __forceinline__ void sharedAdd(float *cell, float v)
{
    asm volatile("red.shared.add.f32 [%0], %1;" :: "r"((unsigned int)__cvta_generic_to_shared(cell)), "f"(v) : "memory");
}

template<typename KeyT, bool HAS_W>
__global__ void __launch_bounds__(TILED_BLOCK, 1)
tiledDeliverKernel(const TiledLaunch L)
{
    extern __shared__ float acc[];
    if(!L.state->heavy) return;
    const unsigned int k = L.state->phase;
    const unsigned int lane = threadIdx.x & 31u;
    const unsigned int warp = threadIdx.x >> 5;
    constexpr unsigned int WARPS = TILED_BLOCK / 32;
    const unsigned int postMask = (1u << L.post_bits) - 1u;
    const KeyT *__restrict__ keys = static_cast<const KeyT*>(L.keys);
    const unsigned int first = L.cta_first_item[blockIdx.x], last = L.cta_first_item[blockIdx.x + 1];
    unsigned int curTile = 0xFFFFFFFFu, curBatch = 0;
    unsigned long long events = 0;

    auto flush = [&]() {
        const TiledTile &T = L.tiles[curTile];
        __syncthreads();
        const unsigned int front = (T.depth > 1u) ? ringSlot(k + 1u, T.depth) : 0u;
        float *base = T.target + (unsigned long long)curBatch * T.depth * T.num_trg + T.first_trg;
        for(unsigned int d = 0; d < T.depth; d++) {
            unsigned int slot = front + d;
            if(slot >= T.depth) slot -= T.depth;
            float *row = base + (unsigned long long)slot * T.num_trg;
            for(unsigned int p = threadIdx.x; p < T.num_tile; p += TILED_BLOCK) {
                const float v = acc[d * T.stride + p];
                if(v != 0.0f) redAdd(row + p, v);
            }
        }
        __syncthreads();
    };

    for(unsigned int item = first; item < last; item++) {
        const unsigned int b = item / L.items_per_batch;
        const unsigned int it = item - b * L.items_per_batch;
        const unsigned int tile = L.item_tile[it];
        const unsigned int share = L.item_share[it];
        if(tile != curTile || b != curBatch) {
            if(curTile != 0xFFFFFFFFu) flush();
            curTile = tile;
            curBatch = b;
            const TiledTile &Z = L.tiles[tile];
            for(unsigned int c = threadIdx.x; c < Z.depth * Z.stride; c += TILED_BLOCK) acc[c] = 0.0f;
            __syncthreads();
        }
        const TiledTile &T = L.tiles[tile];
        for(unsigned int si = 0; si < T.num_sources; si++) {
            const TiledSource &S = L.sources[T.first_source + si];
            const unsigned int slots = S.src_delay_slots;
            const unsigned int rslot = ringSlot(k + slots - S.axonal_delay, slots);
            const unsigned int count = S.spk_cnt[b * slots + rslot];
            const unsigned int *__restrict__ spk = S.spk + ((unsigned long long)b * slots + rslot) * S.num_src;
            const unsigned int *__restrict__ runs = L.run_start + T.table + S.row_base;
            const float cw = S.const_weight;
            // 32 spikes per warp at a time; the spike list is dealt in such batches to the shares, then to the warps
            for(unsigned int q = share + TILED_SPLIT * warp; q * 32u < count; q += TILED_SPLIT * WARPS) {
                const unsigned int i = q * 32u + lane;
                unsigned int a = 0, len = 0;
                if(i < count) {
                    const unsigned int pre = spk[i];
                    if(pre < S.num_src) {
                        a = runs[pre];
                        len = runs[pre + 1] - a;
                    }
                }
                // exclusive prefix sums of the run lengths
                unsigned int incl = len;
#pragma unroll
                for(int o = 1; o < 32; o <<= 1) {
                    const unsigned int up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                    if(lane >= (unsigned int)o) incl += up;
                }
                const unsigned int excl = incl - len;
                const unsigned int total = __shfl_sync(0xFFFFFFFFu, incl, 31);
                events += (lane == 0) ? total : 0u;
#pragma unroll 2
                for(unsigned int x0 = 0; x0 < total; x0 += 32u) {
                    const unsigned int x = x0 + lane;
                    // the run that holds element x: the last one whose exclusive sum is <= x
                    unsigned int lo = 0;
#pragma unroll
                    for(unsigned int s = 16; s > 0; s >>= 1) {
                        const unsigned int v = __shfl_sync(0xFFFFFFFFu, excl, lo + s);
                        if(v <= x) lo += s;
                    }
                    const unsigned int ra = __shfl_sync(0xFFFFFFFFu, a, lo);
                    const unsigned int re = __shfl_sync(0xFFFFFFFFu, excl, lo);
                    if(x < total) {
                        const unsigned int pos = ra + (x - re);
                        const unsigned int key = keys[pos];
                        const float w = HAS_W ? L.weights[pos] : cw;
                        sharedAdd(&acc[(key >> L.post_bits) * T.stride + (key & postMask)], w);
                    }
                }
            }
        }
    }
    if(curTile != 0xFFFFFFFFu) flush();
    if(L.count_events && lane == 0 && events) atomicAdd(&L.state->synaptic_events, events);
}
}   // namespace b200
