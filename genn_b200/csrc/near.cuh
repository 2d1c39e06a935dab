// Near-synapse tables of the warp-specialised kernel's "deliver at emission" mode.
//
// A synapse whose dendritic delay is 0 or 1 step (modulo the ring length: the
// ring index is (front + d) mod D, as in the reference,
// presynapticUpdateStrategySIMT.cc:57-389) is "near": its weight is needed by
// one of the next two neuron updates.  For a cortical model that is one to
// three synapses in a hundred.  These kernels copy the near synapses of ALL
// SPARSE groups into one table keyed by the spiking neuron (one row per neuron
// of every source population, whatever group the synapse belongs to):
//
//     entry = (target index << 8 | ring << 1 | delay (0 or 1),  weight bits)
//
// where `ring` numbers the dendritic-delay rings of the model (one per
// postsynaptic model of a neuron group).  Rows of one source population have a
// fixed power-of-two length (its longest row, rounded up) and are padded with
// zero entries, so the id of a spiking neuron leads to its entries in ONE
// memory round trip, with no row length or offset to fetch first.
//
// The thread that makes a neuron spike delivers these few synapses itself,
// inside the neuron update, straight into the ring slots of the next two steps:
// they are in place when the grid barrier that ends the step completes, and no
// second barrier is needed between "spikes known" and "next neuron update".
// Everything else has two steps of slack and is streamed by other warps.
// The table is a private copy; it is rebuilt whenever the arrays it came from
// may have changed.
#pragma once

#include "common.cuh"

namespace b200
{
// One dendritic-delay ring: den_delay[D][num_neurons] of a postsynaptic model.
struct NearRing
{
    float *den_delay;
    unsigned int D;
    unsigned int num_neurons;
};

// Where the rows of one neuron group's spikes are (a group that is no spike source: shift 0xFFFFFFFF).
// In a sharded model a row holds the synapses onto EVERY process's neurons, one block of
// 1 << peer_shift entries per process (process p: entries [p << peer_shift, (p + 1) << peer_shift)),
// and only the rows of this process's own neurons are here.
struct NearSpace
{
    const uint2 *rows;               // first entry of the row of neuron `first_row`
    unsigned int shift;              // rows hold 1 << shift entries
    unsigned int first_row;          // neuron id of the first row held
    unsigned int peer_shift;         // one process's block of a row (one process: = shift)
    unsigned int pad;
};

constexpr unsigned int NEAR_MAX_RINGS = 64;

// Sharded model: near synapses onto ANOTHER process's neurons travel as 64-bit words (weight bits << 32 | entry
// word) through queues in that process's exchange arena, one queue per (step parity, sending process, sending
// CTA).  Word 0 of a queue is its header, (step << 32 | number of entries), written once the CTA's chain warps are
// through the step; the entries follow from word 1.  The receiving process's CTA of the same index waits for the
// header, takes every entry as soon as it is non-zero (an entry's weight bits are never zero), adds it into its own
// rings and zeroes the word again.  No fence is needed on either side: every word validates itself.  A CTA that
// produces more entries than a queue holds reduces the rest straight into the other process's rings and fences
// before it sends the header.
constexpr unsigned int NEAR_QUEUE_WORDS = 2048;     // default capacity of one queue, header included (16 KB)
constexpr unsigned int NEAR_QUEUE_COUNT = 160;      // queues per (parity, sending process): at least the grid size

struct NearOutbox
{
    unsigned long long *queue[B200_MAX_RANKS];      // this CTA's queue of step parity 0 in every process's arena
    unsigned int count[B200_MAX_RANKS];             // entries queued for each process in the current step
    unsigned int words;                             // capacity of a queue, header included; 0: no queues
    unsigned int fenced;                            // an entry went the direct way: fence before the header
    unsigned long long parity_words;                // distance between the queues of parity 0 and 1, in words
};

__device__ __forceinline__ unsigned int nearDelay(unsigned int d, unsigned int D)
{
    return d % D;
}

// counts[row] += near synapses of the row.  One warp per row.
__global__ void nearCountKernel(const b200_synapse_group g, unsigned int *counts)
{
    const unsigned int lane = threadIdx.x & 31u, warps = blockDim.x >> 5;
    const unsigned int D = g.max_den_delay;
    for(unsigned int row = blockIdx.x * warps + (threadIdx.x >> 5); row < g.num_src; row += gridDim.x * warps) {
        const unsigned int n = min(g.row_length[row], g.row_stride);
        const uint8_t *d = g.d + (unsigned long long)row * g.row_stride;
        unsigned int c = 0;
        for(unsigned int j = lane; j < n; j += 32u) c += (nearDelay(d[j], D) < 2u) ? 1u : 0u;
        #pragma unroll
        for(int o = 16; o; o >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, o);
        if(lane == 0 && c) atomicAdd(&counts[row], c);      // several groups may share the row
    }
}

// Append the row's near synapses to its row of the table (cursor[row] counts what is there).
template<typename IndT>
__global__ void nearFillKernel(const b200_synapse_group g, unsigned int ring, unsigned int *cursor, uint2 *rows,
                               unsigned int shift, unsigned int *bad)
{
    const unsigned int lane = threadIdx.x & 31u, warps = blockDim.x >> 5;
    const unsigned int D = g.max_den_delay;
    const bool constantWeight = (g.wu_model == B200_WU_STATIC_PULSE_CONSTANT_WEIGHT);
    for(unsigned int row = blockIdx.x * warps + (threadIdx.x >> 5); row < g.num_src; row += gridDim.x * warps) {
        const unsigned int n = min(g.row_length[row], g.row_stride);
        const unsigned long long rowStart = (unsigned long long)row * g.row_stride;
        for(unsigned int j0 = 0; j0 < n; j0 += 32u) {
            const unsigned int j = j0 + lane;
            unsigned int e = 2u;
            if(j < n) e = nearDelay(g.d[rowStart + j], D);
            const bool take = e < 2u;
            const unsigned int ballot = __ballot_sync(0xFFFFFFFFu, take);
            if(!ballot) continue;
            unsigned int base = 0;
            if(lane == 0) base = atomicAdd(&cursor[row], (unsigned int)__popc(ballot));
            base = __shfl_sync(0xFFFFFFFFu, base, 0);
            if(take) {
                const unsigned int post = static_cast<const IndT*>(g.ind)[rowStart + j];
                const unsigned int pos = base + __popc(ballot & ((1u << lane) - 1u));
                if(post >= g.num_trg || post >= (1u << 24) || pos >= (1u << shift)) {
                    atomicOr(bad, 1u);
                }
                else {
                    const float w = constantWeight ? g.wu_params[0] : g.g[rowStart + j];
                    rows[((unsigned long long)row << shift) + pos] = make_uint2((post << 8) | (ring << 1) | e, __float_as_uint(w));
                }
            }
        }
    }
}

// The near synapses of one spiking neuron, delivered by its warp: one memory round trip for the
// whole row (`row`: its first entry), up to eight loads per lane in flight.  In a sharded model the
// row has one block per process and `rings` one set of rings per process, the other processes'
// mapped here: reductions into those travel over NVLink.  `front` is the phase of the step in
// which the neuron spiked: a synapse of delay e lands in the slot the neuron update e + 1 steps
// later reads.  With an outbox (`box`), entries for another process go into this CTA's queue in that
// process's arena.  Returns non-zero if a ring of another process was written directly: the caller then owes a
// system-wide fence before that process is told the step is complete.  (Measured on two GPUs: that
// fence costs a spiking warp 7.2 k cycles behind about 50 reductions; making the additions with
// atomics that return the old value and consuming the returns instead cost 9.6 k, they do not overlap.)
template<bool SHARDED>
__device__ __forceinline__ float nearDeliverRow(const uint2 *__restrict__ row, unsigned int shift, unsigned int peerShift,
                                               const NearRing *rings, unsigned int numRings, unsigned int rank,
                                               unsigned int front, StepState *state,
                                               NearOutbox *box = nullptr, unsigned int parity = 0u)
{
    const unsigned int lane = threadIdx.x & 31u;
    const unsigned int cells = 1u << shift;
    float returned = 0.0f;
    for(unsigned int c0 = 0; c0 < cells; c0 += 256u) {
        // up to eight loads per lane in flight before the first reduction
        uint2 entry[8];
        #pragma unroll
        for(unsigned int u = 0; u < 8u; u++) {
            const unsigned int c = c0 + u * 32u + lane;
            entry[u] = (c < cells) ? __ldg(&row[c]) : make_uint2(0u, 0u);
        }
        #pragma unroll
        for(unsigned int u = 0; u < 8u; u++) {
            if(entry[u].y != 0u) {
                // whose neurons this block of the row targets: that process's rings, as mapped here
                // (one process: everything is its own; spelled out because the extra work below sits on
                // the step's critical path)
                const unsigned int owner = SHARDED ? ((c0 + u * 32u + lane) >> peerShift) : rank;
                const unsigned int word = entry[u].x;
                const NearRing &ring = rings[owner * numRings + ((word >> 1) & 0x7Fu)];
                const unsigned int post = word >> 8;
                if(post < ring.num_neurons) {
                    if(SHARDED && owner != rank && box && box->words) {
                        const unsigned int pos = atomicAdd(&box->count[owner], 1u);
                        if(pos + 1u < box->words) {
                            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::
                                         "l"(box->queue[owner] + parity * box->parity_words + 1u + pos),
                                         "l"(((unsigned long long)entry[u].y << 32) | word) : "memory");
                            continue;
                        }
                        box->fenced = 1u;
                    }
                    float *cell = ring.den_delay + (unsigned long long)ringSlot(front + 2u + (word & 1u), ring.D) * ring.num_neurons + post;
                    redAdd(cell, __uint_as_float(entry[u].y));
                    if(SHARDED && owner != rank) returned = 1.0f;
                }
                else {
                    atomicOr(&state->error, ERR_IND_RANGE);
                }
            }
        }
    }
    return returned;
}
}   // namespace b200
