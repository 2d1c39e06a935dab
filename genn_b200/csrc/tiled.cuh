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
// Work: 148 CTAs x 1024 threads, one per SM.  The unit of work is a batch of 32 spikes of one
// source group into one tile.  tiledDecideKernel, one CTA launched before, lays all batches of
// the step out on a line in (batch element, tile, source) order, each weighted with the mean
// run length of its (tile, source) pair, and cuts the line into 148 equally heavy stretches
// from the ACTUAL spike counts of the step; a CTA therefore touches one or two tiles (zeroed
// and flushed once each) whatever the firing pattern.  Inside a stretch the warps draw batch
// tickets from a shared-memory counter; a warp reads the 32 run bounds of its batch and walks
// the concatenation of the runs with all lanes busy (run found by a shuffle search over the
// prefix sums), four rounds of loads in flight.
//
// A step with few events is cheaper on the one-reduction-per-event kernel (no tile to zero
// and flush); tiledDecideKernel estimates the step's events from the spike counts first and
// both delivery kernels obey its verdict.
#pragma once

#include "common.cuh"

namespace b200
{
constexpr int TILED_BLOCK = 1024;
constexpr unsigned int TILED_ACC_FLOATS = 45056;       // 176 KB of accumulators per CTA
constexpr unsigned int TILED_UNROLL = 4;               // rounds of 32 events whose loads are in flight together
constexpr unsigned int TILED_MAX_SOURCES = 64;         // synapse groups onto one target buffer

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

struct TiledPair                // a (tile, source group) pair: the unit the step's work is laid out in
{
    unsigned short tile;
    unsigned short source;      // index into the tile's sources
    float mean_run;             // synapses of the pair per source neuron
};

struct TiledLaunch
{
    const TiledTile *tiles;
    const TiledSource *sources;
    const TiledPair *pairs;             // [num_pairs], tile-major
    const unsigned int *run_start;      // [entries]: absolute position of every (tile, row) run
    const void *keys;
    const float *weights;               // NULL: constant weights
    // written by tiledDecideKernel every heavy step
    unsigned int *pair_batches;         // [batch * num_pairs]: batches of 32 spikes of the pair in this step
    double *pair_prefix;                // [batch * num_pairs]: inclusive prefix of the expected events
    unsigned int *cta_start;            // [(grid + 1) * 2]: (pair, batch) where the stretch of each CTA begins
    unsigned int num_pairs;
    unsigned int num_sources;
    unsigned int grid;
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
__device__ __forceinline__ unsigned int tiledSpikeCount(const TiledSource &S, unsigned int b, unsigned int k)
{
    const unsigned int rslot = ringSlot(k + S.src_delay_slots - S.axonal_delay, S.src_delay_slots);
    return S.spk_cnt[b * S.src_delay_slots + rslot];
}

// One CTA.  Estimates the synaptic events of the step from the spike counts; the verdict is read by
// the tiled kernel and by the one-reduction-per-event kernel.  For a heavy step it also lays the
// step's batches out and cuts them into one stretch per CTA of the tiled kernel.
__global__ void __launch_bounds__(TILED_BLOCK)
tiledDecideKernel(const TiledLaunch L)
{
    __shared__ double chunk[TILED_BLOCK];
    __shared__ float partial[32];
    __shared__ unsigned int verdict;
    const unsigned int k = L.state->phase;
    float est = 0.0f;
    for(unsigned int i = threadIdx.x; i < L.num_sources * L.batch; i += TILED_BLOCK) {
        const TiledSource &s = L.sources[i / L.batch];
        est += (float)tiledSpikeCount(s, i % L.batch, k) * s.mean_row;
    }
    for(int o = 16; o > 0; o >>= 1) est += __shfl_xor_sync(0xFFFFFFFFu, est, o);
    if((threadIdx.x & 31u) == 0) partial[threadIdx.x >> 5] = est;
    __syncthreads();
    if(threadIdx.x == 0) {
        float sum = 0.0f;
        for(unsigned int w = 0; w < TILED_BLOCK / 32; w++) sum += partial[w];
        verdict = (sum >= L.min_events) ? 1u : 0u;
        L.state->heavy = verdict;
    }
    __syncthreads();
    if(!verdict) return;

    // expected events of every (batch element, pair), inclusive prefix over all of them
    const unsigned int total = L.num_pairs * L.batch;
    const unsigned int per = (total + TILED_BLOCK - 1) / TILED_BLOCK;
    const unsigned int lo = min(total, threadIdx.x * per), hi = min(total, lo + per);
    double run = 0.0;
    for(unsigned int p = lo; p < hi; p++) {
        const TiledPair &P = L.pairs[p % L.num_pairs];
        const TiledSource &S = L.sources[L.tiles[P.tile].first_source + P.source];
        const unsigned int nb = (tiledSpikeCount(S, p / L.num_pairs, k) + 31u) / 32u;
        L.pair_batches[p] = nb;
        run += (double)nb * (double)(32.0f * P.mean_run + 64.0f);       // + the fixed cost of a batch
        L.pair_prefix[p] = run;
    }
    chunk[threadIdx.x] = run;
    __syncthreads();
    for(unsigned int o = 1; o < TILED_BLOCK; o <<= 1) {
        const double v = (threadIdx.x >= o) ? chunk[threadIdx.x - o] : 0.0;
        __syncthreads();
        chunk[threadIdx.x] += v;
        __syncthreads();
    }
    const double before = chunk[threadIdx.x] - run;
    for(unsigned int p = lo; p < hi; p++) L.pair_prefix[p] += before;
    __syncthreads();
    const double all = chunk[TILED_BLOCK - 1];
    for(unsigned int c = threadIdx.x; c <= L.grid; c += TILED_BLOCK) {
        unsigned int pair = total, start = 0;
        if(c < L.grid && all > 0.0) {
            const double target = all * (double)c / (double)L.grid;
            unsigned int a = 0, b = total;          // first pair whose inclusive prefix exceeds the target
            while(a < b) {
                const unsigned int m = (a + b) >> 1;
                if(L.pair_prefix[m] > target) b = m; else a = m + 1;
            }
            pair = a;
            if(pair < total) {
                const double prev = pair ? L.pair_prefix[pair - 1] : 0.0;
                const double w = L.pair_prefix[pair] - prev;
                const unsigned int nb = L.pair_batches[pair];
                start = (w > 0.0) ? min(nb, (unsigned int)((target - prev) / w * (double)nb)) : 0u;
            }
        }
        L.cta_start[2 * c] = pair;
        L.cta_start[2 * c + 1] = start;
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
    __shared__ unsigned int pieceStart[TILED_MAX_SOURCES + 1];      // batch tickets before each piece of the segment
    __shared__ unsigned int piecePair[TILED_MAX_SOURCES], pieceLow[TILED_MAX_SOURCES];
    __shared__ unsigned int numPieces, nextTicket, segmentEnd;
    if(!L.state->heavy) return;
    const unsigned int k = L.state->phase;
    const unsigned int lane = threadIdx.x & 31u;
    const unsigned int postMask = (1u << L.post_bits) - 1u;
    const KeyT *__restrict__ keys = static_cast<const KeyT*>(L.keys);
    const unsigned int p0 = L.cta_start[2 * blockIdx.x], b0 = L.cta_start[2 * blockIdx.x + 1];
    const unsigned int p1 = L.cta_start[2 * blockIdx.x + 2], b1 = L.cta_start[2 * blockIdx.x + 3];
    unsigned long long events = 0;

    // a segment: the pieces (pair, batch range) of this CTA's stretch that lie in ONE tile of one batch element
    unsigned int p = p0;
    while(p < p1 || (p == p1 && b1 > 0u)) {
        const unsigned int b = p / L.num_pairs;
        const unsigned int tile = L.pairs[p - b * L.num_pairs].tile;
        const TiledTile &T = L.tiles[tile];
        if(threadIdx.x < 32u) {
            // warp 0 lists the pieces of the segment, one lane per candidate pair
            unsigned int n = 0, before = 0;
            for(unsigned int q0 = p;; q0 += 32u) {
                const unsigned int q = q0 + lane;
                const bool in = (q < p1 || (q == p1 && b1 > 0u)) && (q / L.num_pairs == b) && (L.pairs[q % L.num_pairs].tile == tile);
                const unsigned int mask = __ballot_sync(0xFFFFFFFFu, in);
                const unsigned int cnt = (mask == 0xFFFFFFFFu) ? 32u : (unsigned int)__ffs(~mask) - 1u;    // the segment is a run of pairs
                unsigned int low = 0, tk = 0;
                if(lane < cnt) {
                    low = (q == p0) ? b0 : 0u;
                    const unsigned int high = (q == p1) ? b1 : L.pair_batches[q];
                    tk = (high > low) ? high - low : 0u;
                }
                unsigned int incl = tk;
#pragma unroll
                for(int o = 1; o < 32; o <<= 1) {
                    const unsigned int up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                    if(lane >= (unsigned int)o) incl += up;
                }
                if(lane < cnt) {
                    pieceStart[n + lane] = before + incl - tk;
                    piecePair[n + lane] = q;
                    pieceLow[n + lane] = low;
                }
                before += __shfl_sync(0xFFFFFFFFu, incl, 31);
                n += cnt;
                if(cnt < 32u) break;
            }
            if(lane == 0) {
                pieceStart[n] = before;
                numPieces = n;
                nextTicket = 0;
                segmentEnd = p + n;
            }
        }
        for(unsigned int c = threadIdx.x; c < T.depth * T.stride; c += TILED_BLOCK) acc[c] = 0.0f;
        __syncthreads();
        const unsigned int tickets = pieceStart[numPieces];
        for(;;) {
            unsigned int ticket = 0;
            if(lane == 0) ticket = atomicAdd(&nextTicket, 1u);
            ticket = __shfl_sync(0xFFFFFFFFu, ticket, 0);
            if(ticket >= tickets) break;
            unsigned int j = 0;
            while(pieceStart[j + 1] <= ticket) j++;
            const unsigned int f = pieceLow[j] + (ticket - pieceStart[j]);
            const TiledSource &S = L.sources[T.first_source + L.pairs[piecePair[j] % L.num_pairs].source];
            const unsigned int slots = S.src_delay_slots;
            const unsigned int rslot = ringSlot(k + slots - S.axonal_delay, slots);
            const unsigned int count = S.spk_cnt[b * slots + rslot];
            const unsigned int *__restrict__ spk = S.spk + ((unsigned long long)b * slots + rslot) * S.num_src;
            const unsigned int *__restrict__ runs = L.run_start + T.table + S.row_base;
            const float cw = S.const_weight;
            const unsigned int i = f * 32u + lane;
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
            // the concatenation of the 32 runs, TILED_UNROLL x 32 elements per round; the loads of round
            // r + 1 are issued before the accumulations of round r (two rounds of loads in flight)
            unsigned int key[TILED_UNROLL], nextKey[TILED_UNROLL];
            float w[TILED_UNROLL], nextW[TILED_UNROLL];
            unsigned int valid = 0, nextValid = 0;      // bit u: element u of the round exists
            auto fetch = [&](unsigned int x0) {
                nextValid = 0;
#pragma unroll
                for(unsigned int u = 0; u < TILED_UNROLL; u++) {
                    const unsigned int x = x0 + u * 32u + lane;
                    // the run that holds element x: the last one whose exclusive sum is <= x
                    unsigned int lo = 0;
#pragma unroll
                    for(unsigned int st = 16; st > 0; st >>= 1) {
                        const unsigned int v = __shfl_sync(0xFFFFFFFFu, excl, lo + st);
                        if(v <= x) lo += st;
                    }
                    const unsigned int ra = __shfl_sync(0xFFFFFFFFu, a, lo);
                    const unsigned int re = __shfl_sync(0xFFFFFFFFu, excl, lo);
                    if(x < total) {
                        const unsigned int pos = ra + (x - re);
                        nextKey[u] = keys[pos];
                        nextW[u] = HAS_W ? L.weights[pos] : cw;
                        nextValid |= 1u << u;
                    }
                }
            };
            if(total) fetch(0);
            for(unsigned int x0 = 0; x0 < total; x0 += 32u * TILED_UNROLL) {
                valid = nextValid;
#pragma unroll
                for(unsigned int u = 0; u < TILED_UNROLL; u++) {
                    key[u] = nextKey[u];
                    w[u] = nextW[u];
                }
                if(x0 + 32u * TILED_UNROLL < total) fetch(x0 + 32u * TILED_UNROLL);
#pragma unroll
                for(unsigned int u = 0; u < TILED_UNROLL; u++) {
                    if(valid & (1u << u)) sharedAdd(&acc[(key[u] >> L.post_bits) * T.stride + (key[u] & postMask)], w[u]);
                }
            }
        }
        // every touched cell goes to L2 once
        __syncthreads();
        {
            const unsigned int front = (T.depth > 1u) ? ringSlot(k + 1u, T.depth) : 0u;
            float *base = T.target + (unsigned long long)b * T.depth * T.num_trg + T.first_trg;
            // a row of the tile in L2 as items of four cells aligned to 16 bytes (one vector reduction each)
            // plus the unaligned cells at its two ends
            const unsigned int itemsPerRow = (T.num_tile + 3u) / 4u + 1u;
            for(unsigned int it = threadIdx.x; it < T.depth * itemsPerRow; it += TILED_BLOCK) {
                const unsigned int d = it / itemsPerRow, i = it - d * itemsPerRow;
                unsigned int slot = front + d;
                if(slot >= T.depth) slot -= T.depth;
                float *row = base + (unsigned long long)slot * T.num_trg;
                const unsigned int lead = min(T.num_tile, (4u - (unsigned int)((reinterpret_cast<unsigned long long>(row) >> 2) & 3ull)) & 3u);
                const float *cells = acc + d * T.stride;
                if(i == 0) {
                    for(unsigned int t = 0; t < lead; t++) {
                        if(cells[t] != 0.0f) redAdd(row + t, cells[t]);
                    }
                }
                else {
                    const unsigned int t = lead + (i - 1u) * 4u;
                    if(t + 4u <= T.num_tile) {
                        const float v0 = cells[t], v1 = cells[t + 1], v2 = cells[t + 2], v3 = cells[t + 3];
                        if(v0 != 0.0f || v1 != 0.0f || v2 != 0.0f || v3 != 0.0f) {
                            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                                         :: "l"(__cvta_generic_to_global(row + t)), "f"(v0), "f"(v1), "f"(v2), "f"(v3) : "memory");
                        }
                    }
                    else {
                        for(unsigned int u = t; u < T.num_tile; u++) {
                            if(cells[u] != 0.0f) redAdd(row + u, cells[u]);
                        }
                    }
                }
            }
        }
        p = segmentEnd;
        __syncthreads();
    }
    if(L.count_events && lane == 0 && events) atomicAdd(&L.state->synaptic_events, events);
}
}   // namespace b200
