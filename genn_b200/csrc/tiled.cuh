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
// Work: 148 CTAs x 1024 threads, one per SM.  The unit of work is a ticket: up to 32 spikes of one source
// group into one tile, fewer where the runs of the (tile, source) pair are long, so that a ticket stays near two
// thousand synaptic events (one warp walks a ticket: with coarser tickets the last ones of a tile ran with the
// other warps idle, a third of the kernel's time).  tiledDecideKernel, one CTA launched before, lays all tickets
// of the step out on a line in (batch element, tile, source) order, each weighted with the mean run length of its
// (tile, source) pair plus a fixed cost, and cuts the line into 148 equally heavy stretches from the ACTUAL spike
// counts of the step; a CTA therefore touches one to three tiles (zeroed and flushed once each) whatever the firing
// pattern.  Inside a stretch the warps draw tickets from a shared-memory counter; a warp reads the run bounds of
// its ticket's spikes and walks the concatenation of the runs with all lanes busy, two rounds of four loads per
// lane in flight.  The run that holds an element is found without a search: the runs that begin inside a window of
// 32 elements make a bit mask (one warp-wide OR), the run of an element is counted from it, its offset read from
// shared memory.
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

// Spikes of a (tile, source group) pair that make one ticket of the tiled kernel: 32, fewer where runs are long, so that
// a ticket stays near a thousand synaptic events (one warp walks a ticket; the last tickets of a tile run with most
// warps idle).
__host__ __device__ __forceinline__ unsigned int tiledTicketSpikes(float meanRun, float ticketEvents)
{
    unsigned int s = 32u;
    while(s > 1u && (float)s * meanRun > ticketEvents) s >>= 1;
    return s;
}

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
    float ticket_events;                // synaptic events a ticket is sized for (tiledTicketSpikes)
    float ticket_cost;                  // fixed cost of a ticket when the step's work is cut into stretches, in synaptic events
    StepState *state;
    unsigned int count_events;
    unsigned long long *profile;        // NULL, or [grid][4]: cycles of the CTA, of them outside the ticket loops; segments << 32 | tickets; cycles the warps idled at the ends of the ticket loops (mean)
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
        const unsigned int spikes = tiledTicketSpikes(P.mean_run, L.ticket_events);
        const unsigned int nb = (tiledSpikeCount(S, p / L.num_pairs, k) + spikes - 1u) / spikes;
        L.pair_batches[p] = nb;
        run += (double)nb * (double)((float)spikes * P.mean_run + L.ticket_cost);
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
    __shared__ unsigned int runOffset[TILED_BLOCK];     // per warp: (start of run - elements before it) of its non-empty runs
    __shared__ unsigned int pieceStart[TILED_MAX_SOURCES + 1];      // batch tickets before each piece of the segment
    __shared__ unsigned int pieceLow[TILED_MAX_SOURCES];
    // what a ticket of the piece needs: the spike list of its source, the run table of (tile, source), the ticket size
    __shared__ const unsigned int *pieceSpk[TILED_MAX_SOURCES], *pieceRuns[TILED_MAX_SOURCES];
    __shared__ unsigned int pieceCount[TILED_MAX_SOURCES], pieceRows[TILED_MAX_SOURCES], pieceSpikes[TILED_MAX_SOURCES];
    __shared__ float pieceWeight[TILED_MAX_SOURCES];
    __shared__ unsigned int numPieces, nextTicket, segmentEnd;
    if(!L.state->heavy) return;
    const unsigned int k = L.state->phase;
    const unsigned int lane = threadIdx.x & 31u;
    const unsigned int postMask = (1u << L.post_bits) - 1u;
    const KeyT *__restrict__ keys = static_cast<const KeyT*>(L.keys);
    const unsigned int p0 = L.cta_start[2 * blockIdx.x], b0 = L.cta_start[2 * blockIdx.x + 1];
    const unsigned int p1 = L.cta_start[2 * blockIdx.x + 2], b1 = L.cta_start[2 * blockIdx.x + 3];
    unsigned long long events = 0;
    // clock64 record of thread 0 (option fused_profile): start, last mark, cycles outside the ticket loops, segments << 32 | tickets
    __shared__ long long prof[5], warpEnd[TILED_BLOCK / 32];
    const bool profiling = (L.profile != nullptr) && (threadIdx.x == 0);
    if(profiling) {
        prof[0] = prof[1] = clock64();
        prof[2] = prof[3] = prof[4] = 0;
    }
    const unsigned int laneLess = (1u << lane) - 1u, laneLessEq = laneLess | (1u << lane);

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
                    pieceLow[n + lane] = low;
                    const TiledPair &P = L.pairs[q % L.num_pairs];
                    const TiledSource &S = L.sources[T.first_source + P.source];
                    const unsigned int slots = S.src_delay_slots;
                    const unsigned int rslot = ringSlot(k + slots - S.axonal_delay, slots);
                    pieceCount[n + lane] = S.spk_cnt[b * slots + rslot];
                    pieceSpk[n + lane] = S.spk + ((unsigned long long)b * slots + rslot) * S.num_src;
                    pieceRuns[n + lane] = L.run_start + T.table + S.row_base;
                    pieceRows[n + lane] = S.num_src;
                    pieceWeight[n + lane] = S.const_weight;
                    pieceSpikes[n + lane] = tiledTicketSpikes(P.mean_run, L.ticket_events);
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
        if(profiling) {
            prof[2] += clock64() - prof[1];
            prof[3] += (1ll << 32) + tickets;
        }
        for(;;) {
            unsigned int ticket = 0;
            if(lane == 0) ticket = atomicAdd(&nextTicket, 1u);
            ticket = __shfl_sync(0xFFFFFFFFu, ticket, 0);
            if(ticket >= tickets) break;
            unsigned int j = 0;
            while(pieceStart[j + 1] <= ticket) j++;
            const unsigned int f = pieceLow[j] + (ticket - pieceStart[j]);
            const unsigned int perTicket = pieceSpikes[j];
            const unsigned int *__restrict__ runs = pieceRuns[j];
            const float cw = pieceWeight[j];
            const unsigned int i = f * perTicket + lane;
            unsigned int a = 0, len = 0;
            if(lane < perTicket && i < pieceCount[j]) {
                const unsigned int pre = pieceSpk[j][i];
                if(pre < pieceRows[j]) {
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
            // The non-empty runs, in order, at the front of the warp's offset table: element x of the
            // concatenation, in run c, lies at x + offset[c] of the tile's arrays.
            unsigned int *offs = runOffset + (threadIdx.x & ~31u);
            const unsigned int nonEmpty = __ballot_sync(0xFFFFFFFFu, len != 0u);
            __syncwarp();                                   // (the previous ticket's reads of the table)
            if(len) offs[__popc(nonEmpty & laneLess)] = a - excl;
            __syncwarp();
            // Non-empty runs begin at distinct elements.  For a window of 32 elements the lanes OR together one
            // bit per run that begins inside it; the run of element j of the window is the number of runs
            // begun before the window plus the bits up to j, minus one.
            const unsigned int head = len ? excl : 0xFFFFFFFFu;
            unsigned int begun = 0;
            struct Round { unsigned int key[TILED_UNROLL]; float w[TILED_UNROLL]; unsigned int valid; };
            auto fetch = [&](Round &R, unsigned int x0) {
                R.valid = 0;
#pragma unroll
                for(unsigned int u = 0; u < TILED_UNROLL; u++) {
                    const unsigned int first = x0 + u * 32u;
                    unsigned int bit;       // (shl gives 0 for a shift of 32 or more: a head before or beyond the window)
                    asm("shl.b32 %0, %1, %2;" : "=r"(bit) : "r"(1u), "r"(head - first));
                    const unsigned int heads = __reduce_or_sync(0xFFFFFFFFu, bit);
                    const unsigned int c = begun + __popc(heads & laneLessEq) - 1u;
                    begun += __popc(heads);
                    const unsigned int x = first + lane;
                    if(x < total) {
                        const unsigned int pos = x + offs[c];
                        R.key[u] = keys[pos];
                        R.w[u] = HAS_W ? L.weights[pos] : cw;
                        R.valid |= 1u << u;
                    }
                }
            };
            auto deliver = [&](const Round &R) {
#pragma unroll
                for(unsigned int u = 0; u < TILED_UNROLL; u++) {
                    if(R.valid & (1u << u)) sharedAdd(&acc[(R.key[u] >> L.post_bits) * T.stride + (R.key[u] & postMask)], R.w[u]);
                }
            };
            // two rounds of loads in flight, in two sets of registers
            constexpr unsigned int ROUND = 32u * TILED_UNROLL;
            Round A, B;
            if(total) fetch(A, 0);
            for(unsigned int x0 = 0; x0 < total; x0 += 2u * ROUND) {
                const bool second = x0 + ROUND < total;
                if(second) fetch(B, x0 + ROUND);
                deliver(A);
                if(!second) break;
                if(x0 + 2u * ROUND < total) fetch(A, x0 + 2u * ROUND);
                deliver(B);
            }
        }
        // every touched cell goes to L2 once
        if(L.profile && lane == 0) warpEnd[threadIdx.x >> 5] = clock64();
        __syncthreads();
        if(profiling) {
            prof[1] = clock64();
            long long last = warpEnd[0], sum = 0;
            for(unsigned int w = 0; w < TILED_BLOCK / 32; w++) {
                last = max(last, warpEnd[w]);
                sum += warpEnd[w];
            }
            prof[4] += last - sum / (TILED_BLOCK / 32);     // cycles the warps idled on average while the last ticket ran
        }
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
    if(profiling) {
        const long long now = clock64();
        unsigned long long *out = L.profile + 4ull * blockIdx.x;
        out[0] = (unsigned long long)(now - prof[0]);
        out[1] = (unsigned long long)(prof[2] + (now - prof[1]));
        out[2] = (unsigned long long)prof[3];
        out[3] = (unsigned long long)prof[4];
    }
}
}   // namespace b200
