// C ABI of the B200 backend (include/genn_b200.h) and the runner behind it.
//
// A runner is the counterpart of one loaded librunner.so of the reference: it
// owns the stream, the device-resident step counters, the merged-group tables
// and the captured step graph.  The time-step path allocates nothing and never
// synchronises; the host only enqueues (one cudaGraphLaunch per block of steps).
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <cctype>
#include <cstdarg>
#include <cstdlib>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "genn_b200.h"
#include "common.cuh"
#include "neuron_update.cuh"
#include "presynaptic_update.cuh"
#include "postsynaptic_update.cuh"
#include "init.cuh"
#include "fused_step.cuh"
#include "urgent.cuh"
#include "stream_step.cuh"
#include "tiled.cuh"

#include <cub/device/device_scan.cuh>

using namespace b200;

namespace
{
thread_local std::string g_lastError;

int fail(int code, const char *fmt, ...)
{
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_lastError = buf;
    return code;
}

#define CUDA_TRY(expr)                                                                           \
    do {                                                                                         \
        cudaError_t _e = (expr);                                                                 \
        if(_e != cudaSuccess) {                                                                  \
            return fail(B200_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),   \
                        __FILE__, __LINE__);                                                     \
        }                                                                                        \
    } while(0)

constexpr size_t ARRAY_TAIL_PAD = 256;     // vector loads may read up to 15 bytes past the last element

template<typename T>
struct DeviceTable
{
    T *d = nullptr;
    unsigned int *blockStart = nullptr;
    unsigned int num = 0;
    unsigned int blocks = 0;

    void release()
    {
        if(d) cudaFree(d);
        if(blockStart) cudaFree(blockStart);
        d = nullptr; blockStart = nullptr; num = 0; blocks = 0;
    }

    cudaError_t upload(const std::vector<T> &items, const std::vector<unsigned int> &starts, cudaStream_t s)
    {
        release();
        num = (unsigned int)items.size();
        if(num == 0) return cudaSuccess;
        blocks = starts.back();
        cudaError_t e = cudaMalloc(&d, sizeof(T) * num);
        if(e != cudaSuccess) return e;
        e = cudaMalloc(&blockStart, sizeof(unsigned int) * starts.size());
        if(e != cudaSuccess) return e;
        e = cudaMemcpyAsync(d, items.data(), sizeof(T) * num, cudaMemcpyHostToDevice, s);
        if(e != cudaSuccess) return e;
        e = cudaMemcpyAsync(blockStart, starts.data(), sizeof(unsigned int) * starts.size(), cudaMemcpyHostToDevice, s);
        if(e != cudaSuccess) return e;
        return cudaStreamSynchronize(s);
    }
};

struct Timer
{
    double seconds = 0.0;
};
}   // anonymous namespace

// Device buffer that is freed on every early return of a build function unless it was handed over.
struct ScopedDevice
{
    void *p = nullptr;
    ~ScopedDevice() { if(p) cudaFree(p); }
    template<typename T> T *as() const { return static_cast<T*>(p); }
    void *release() { void *q = p; p = nullptr; return q; }
};

constexpr unsigned int PROFILE_MAX_CTAS = 1024;     // per-CTA cycle counters of option "fused_profile"

struct b200_runner
{
    int device = 0;
    float dt = 0.1f;
    unsigned long long seed = 0;
    unsigned int batch = 1;
    cudaStream_t stream = nullptr;
    StepState *state = nullptr;
    std::unordered_map<void*, size_t> arrays;

    std::vector<b200_neuron_group> neuronGroups;
    std::vector<b200_synapse_group> synapseGroups;
    std::map<std::string, std::vector<b200_custom_update_group>> customUpdates;
    bool dirty = true;

    DeviceTable<b200_neuron_group> neuronTable;
    DeviceTable<b200_synapse_group> sparseTable, postSpanTable, learnTable, proceduralTable;

    // persistent fused-step path (batch 1, SPARSE non-learning groups only)
    bool fusedEligible = false;
    bool useFused = true;
    unsigned int fusedBlocksPerSM = 0;      // 0: as many as fit (occupancy query)
    unsigned int fusedGrid = 0;
    unsigned int *fusedSlotStart = nullptr;
    FusedSource *fusedSources = nullptr;
    uint2 *fusedItems = nullptr;
    unsigned int fusedNumSources = 0;
    unsigned int fusedNumItems = 0;
    size_t fusedSmemBytes = 0;
    bool fusedStage = false;
    const void *fusedKernel = nullptr;
    int fusedPerSM = 0;
    unsigned long long *fusedBarrier = nullptr;
    unsigned long long fusedLaunches = 0;
    bool fusedProfile = false;
    unsigned long long *fusedCtaCycles = nullptr;
    // one-step lag of the persistent kernel (fused_step.cuh): allowed while every
    // synapse has a dendritic delay of at least one step
    bool useLag = true;
    bool lagAgreed = false;         // sharded model: the host checked that every process is eligible
    bool lagStale = true;           // delay arrays may have changed since the last scan
    bool lagEligible = false;
    unsigned int *lagScan = nullptr;
    std::vector<b200_synapse_group> fusedGroups;    // host copy of the SPARSE groups the kernel serves
    // split delivery (fused_step.cuh): private tables of the synapses that arrive in the same step
    bool useSplit = true;
    int streamWarpsWanted = -1;                     // -1: as many as the neuron slots leave free, 0: none
    unsigned int streamWarps = 0;                   // of the current tables (0: fusedStepKernel)
    unsigned int slotsPerCta = 0;
    std::vector<unsigned int> urgentStride;         // per SPARSE group: its longest urgent row (0: none)
    unsigned int *urgentOffsets = nullptr;          // row offsets of all groups, one after the other
    uint2 *urgentEntries = nullptr;
    FusedUrgent *fusedUrgent = nullptr;             // device copy for the kernel, or NULL
    enum Schedule { PLAIN = 0, SPLIT = 1, LAG = 2, EMIT = 3 };
    // "deliver at emission" mode (near.cuh): near synapses of all groups, one row per source neuron
    bool useEmit = true;
    uint2 *nearTable = nullptr;             // rows of every source neuron (synapses onto THIS process's neurons)
    NearRing *nearRings = nullptr;          // device copies, [world][numRings] and [world][neuron groups]
    NearSpace *nearSpaces = nullptr;
    unsigned int numRings = 0;
    // sharded model: built by b200_near_export / b200_near_import / b200_near_finish
    std::vector<NearRing> nearRingsHost;            // this process's rings
    std::vector<unsigned long long> nearCellHost;   // per neuron group: first entry of its rows in nearTable
    std::vector<unsigned int> nearShiftHost;        // per neuron group: row length shift (0xFFFFFFFF: no rows)
    std::vector<uint2*> nearImported;               // per neuron group: the rows of this process's neurons, one block per process
    std::vector<NearSpace> nearSpacesAll;           // [neuron groups]
    std::vector<bool> nearPeerDone;                 // per process: its blocks have been copied in
    bool emitAgreed = false;                        // every process exported, imported and qualified
    bool nearDataStale = false;                     // synapse arrays changed after the exchange
    Schedule schedule = PLAIN;

    void dropNear()
    {
        if(nearTable) cudaFree(nearTable);
        if(nearRings) cudaFree(nearRings);
        if(nearSpaces) cudaFree(nearSpaces);
        for(uint2 *p : nearImported) if(p) cudaFree(p);
        nearImported.clear();
        nearTable = nullptr; nearRings = nullptr; nearSpaces = nullptr; numRings = 0;
        emitAgreed = false;
    }

    void dropUrgent()
    {
        urgentStride.clear();
        if(urgentOffsets) cudaFree(urgentOffsets);
        if(urgentEntries) cudaFree(urgentEntries);
        if(fusedUrgent) cudaFree(fusedUrgent);
        urgentOffsets = nullptr; urgentEntries = nullptr; fusedUrgent = nullptr;
        if(!emitAgreed) dropNear();
    }

    // spike exchange of a sharded model
    unsigned char *arena = nullptr;
    size_t arenaBytes = 0;
    // data-parallel runs: communicator for the all-reduce inside batch-reduce custom updates, and the
    // buffer the reduced values of a group are packed into for it
    void *ncclComm = nullptr;
    unsigned int ncclWorld = 1;
    float *reducePacked = nullptr;
    size_t reducePackedElements = 0;
    // queues for near synapses between processes (near.cuh), behind the caller's part of the arena
    size_t queueOffset = 0;
    unsigned int queueWords = NEAR_QUEUE_WORDS;
    bool useNearQueues = true;
    bool queuesAgreed = false;                  // every process runs the same grid, which the queues are numbered by
    unsigned int peerGrid[B200_MAX_RANKS] = {};
    unsigned char *peerArena[B200_MAX_RANKS] = {};
    bool peerLocal[B200_MAX_RANKS] = {};    // mapped by pointer (same process): nothing to close
    unsigned char **peerTable = nullptr;     // device copy of peerArena
    unsigned int rank = 0, world = 1;
    size_t flagsOffset = 0;
    bool sharded() const { return world > 1; }

    // target-tiled delivery of heavy steps on the one-launch-per-kernel path (tiled.cuh): private
    // re-packed copy of the non-learning SPARSE groups
    bool useTiled = true;
    float tiledTicketEvents = 2048.0f, tiledTicketCost = 256.0f;     // (swept on Potjans x1 with a quarter of the neurons spiking)
    float tiledMinEvents = 1.0e6f;          // estimated events of a step from which the tiled kernel takes it
    bool tiledReady = false, tiledStale = true;
    // The tiled kernels cost two launches per step even when they find nothing to do, so they are only
    // launched ("armed") while the network's recent activity could reach the threshold: the neuron kernel
    // keeps the largest spike count of a step in StepState::peak_spikes, the host fetches it (asynchronously,
    // into page-locked memory) behind every block of steps and looks at it before the next block
    bool tiledArmed = false;
    unsigned int *peakHost = nullptr;
    cudaEvent_t peakEvent = nullptr;
    bool peakPending = false;
    unsigned int quietBlocks = 0;
    double eventsPerSpike = 0.0;
    std::string tiledWhyNot;
    TiledTile *tiledTiles = nullptr;
    TiledSource *tiledSources = nullptr;
    unsigned int *tiledRunStart = nullptr, *tiledCtaStart = nullptr, *tiledPairBatches = nullptr;
    void *tiledKeys = nullptr;
    float *tiledWeights = nullptr;
    TiledPair *tiledPairs = nullptr;
    double *tiledPairPrefix = nullptr;
    unsigned char *tiledServed = nullptr;
    unsigned int tiledNumPairs = 0, tiledNumSources = 0, tiledPostBits = 10, tiledGrid = 0;
    size_t tiledSmemBytes = 0;
    unsigned long long tiledSynapses = 0;

    void dropTiled()
    {
        void *bufs[] = {tiledTiles, tiledSources, tiledRunStart, tiledCtaStart, tiledPairBatches, tiledKeys, tiledWeights,
                        tiledPairs, tiledPairPrefix, tiledServed};
        for(void *b : bufs) if(b) cudaFree(b);
        tiledTiles = nullptr; tiledSources = nullptr; tiledRunStart = nullptr; tiledCtaStart = nullptr;
        tiledPairBatches = nullptr; tiledKeys = nullptr; tiledWeights = nullptr; tiledPairs = nullptr;
        tiledPairPrefix = nullptr; tiledServed = nullptr;
        tiledReady = false;
    }

    // options
    unsigned int spikeLanes = 16;
    bool countEvents = false;
    bool useGraph = true;
    unsigned int graphSteps = 100;
    bool timing = false;

    // captured graph of `graphLen` steps for a given recording length
    cudaGraphExec_t graphExec = nullptr;
    unsigned int graphLen = 0;
    unsigned long long graphNumRec = 0;

    std::map<std::string, Timer> timers;
    cudaEvent_t evA = nullptr, evB = nullptr, evC = nullptr, evD = nullptr;
    unsigned long long launches = 0;
    unsigned long long hostTimestep = 0, hostStepsDone = 0;

    void dropGraph()
    {
        if(graphExec) cudaGraphExecDestroy(graphExec);
        graphExec = nullptr;
        graphLen = 0;
    }
};

namespace
{
template<typename F>
int withIndType(unsigned int bytes, F f)
{
    switch(bytes) {
    case 1: return f(uint8_t());
    case 2: return f(uint16_t());
    case 4: return f(uint32_t());
    default: return fail(B200_ERR_INVALID, "index width %u is not 1, 2 or 4", bytes);
    }
}

// Kernel instances by (max fused postsynaptic models, max current sources) of
// any neuron group: the smallest covering instance is used.
struct NeuronShape { int npsm, ncs; };

NeuronShape neuronShape(const b200_runner *r)
{
    unsigned int p = 0, c = 0;
    for(const auto &g : r->neuronGroups) {
        p = std::max(p, g.num_psm);
        c = std::max(c, g.num_cs);
    }
    NeuronShape s;
    s.npsm = (p <= 1) ? 1 : (p <= 2) ? 2 : B200_MAX_PSM;
    s.ncs = (c == 0) ? 0 : (c == 1) ? 1 : B200_MAX_CS;
    return s;
}

template<typename F>
int withNeuronShape(const b200_runner *r, F f)
{
    const NeuronShape s = neuronShape(r);
#define B200_SHAPE(P, C) if(s.npsm == P && s.ncs == C) return f(std::integral_constant<int, P>(), std::integral_constant<int, C>())
    B200_SHAPE(1, 0); B200_SHAPE(1, 1); B200_SHAPE(1, B200_MAX_CS);
    B200_SHAPE(2, 0); B200_SHAPE(2, 1); B200_SHAPE(2, B200_MAX_CS);
    B200_SHAPE(B200_MAX_PSM, 0); B200_SHAPE(B200_MAX_PSM, 1); B200_SHAPE(B200_MAX_PSM, B200_MAX_CS);
#undef B200_SHAPE
    return fail(B200_ERR_INVALID, "no kernel instance for this neuron shape");
}


// Tables of the persistent fused-step kernel for the current schedule: spike
// sources, the two item lists of each, thread slots, shared-memory budget, grid.
int buildFusedTables(b200_runner *r)
{
    if(r->fusedSlotStart) { cudaFree(r->fusedSlotStart); r->fusedSlotStart = nullptr; }
    if(r->fusedSources) { cudaFree(r->fusedSources); r->fusedSources = nullptr; }
    if(r->fusedItems) { cudaFree(r->fusedItems); r->fusedItems = nullptr; }
    if(!r->fusedEligible) return B200_OK;
    const std::vector<b200_synapse_group> &sparse = r->fusedGroups;
    std::vector<unsigned int> slotStart{0};
    for(const auto &g : r->neuronGroups) slotStart.push_back(slotStart.back() + ((g.num_update + 31u) & ~31u));
    std::vector<FusedSource> sources;
    std::vector<std::vector<uint2>> perSource;
    std::vector<std::vector<uint2>> perSourceUrgent;
    for(size_t gi = 0; gi < sparse.size(); gi++) {
        const auto &g = sparse[gi];
        // which list the group's full-row chunks go to, and whether it has a table of urgent synapses
        const bool ring = g.max_den_delay >= 2 && g.d;
        const bool later = (r->schedule == b200_runner::LAG) || (r->schedule == b200_runner::EMIT) ||
                           (r->schedule == b200_runner::SPLIT && ring);
        const unsigned int urgentStride = (r->schedule == b200_runner::SPLIT && gi < r->urgentStride.size())
            ? r->urgentStride[gi] : 0u;
        // a sharded source population contributes one source per process section
        const unsigned int sections = std::max(1u, g.src_sections);
        const unsigned int chunks = (g.row_stride + 3 + FUSED_CHUNK - 1) / FUSED_CHUNK;
        for(unsigned int sec = 0; sec < sections; sec++) {
            const unsigned int *cntPtr = g.src_spk_cnt + sec * g.src_cnt_section_stride;
            size_t si = 0;
            for(; si < sources.size(); si++) {
                if(sources[si].spk_cnt == cntPtr && sources[si].delay == g.axonal_delay) break;
            }
            if(si == sources.size()) {
                FusedSource src{};
                src.spk_cnt = cntPtr;
                src.spk = g.src_spk + sec * g.src_spk_section_stride;
                src.num_src = g.src_spk_slot_stride ? g.src_spk_slot_stride : g.num_src;   // list capacity
                src.slots = g.src_delay_slots;
                src.delay = g.axonal_delay;
                src.spk_tag = g.src_spk_tag
                    ? reinterpret_cast<const unsigned long long*>(g.src_spk_tag + sec * g.src_cnt_section_stride) : nullptr;
                src.spk_wire = g.src_spk_wire
                    ? reinterpret_cast<const unsigned long long*>(g.src_spk_wire + sec * g.src_spk_section_stride) : nullptr;
                sources.push_back(src);
                perSource.emplace_back();
                perSourceUrgent.emplace_back();
            }
            auto &rows = later ? perSource[si] : perSourceUrgent[si];
            for(unsigned int c = 0; c < chunks; c++) rows.push_back(make_uint2((unsigned int)gi, c));
            for(unsigned int c = 0; c < (urgentStride + 31u) / 32u; c++) {
                perSourceUrgent[si].push_back(make_uint2((unsigned int)gi, c | FUSED_URGENT_TABLE));
            }
        }
    }
    std::vector<uint2> items;
    for(size_t si = 0; si < sources.size(); si++) {
        sources[si].item_begin = (unsigned int)items.size();
        sources[si].item_count = (unsigned int)perSource[si].size();
        items.insert(items.end(), perSource[si].begin(), perSource[si].end());
        sources[si].urgent_begin = (unsigned int)items.size();
        sources[si].urgent_count = (unsigned int)perSourceUrgent[si].size();
        items.insert(items.end(), perSourceUrgent[si].begin(), perSourceUrgent[si].end());
    }
    if(sources.size() > FUSED_MAX_SOURCES) {
        return fail(B200_ERR_INVALID, "%zu spike sources exceed the %u the persistent kernel handles",
                    sources.size(), (unsigned int)FUSED_MAX_SOURCES);
    }
    r->fusedNumSources = (unsigned int)sources.size();
    r->fusedNumItems = (unsigned int)items.size();
    r->fusedSmemBytes = align16(sizeof(b200_neuron_group) * r->neuronGroups.size()) +
                        align16(sizeof(b200_synapse_group) * sparse.size()) +
                        align16(sizeof(FusedSource) * sources.size()) + align16(sizeof(uint2) * items.size()) +
                        align16(sizeof(unsigned int) * slotStart.size()) +
                        (r->fusedUrgent ? align16(sizeof(FusedUrgent) * sparse.size()) : 0) +
                        (r->schedule == b200_runner::EMIT
                            ? align16(sizeof(NearRing) * r->numRings * r->world) +
                              align16(sizeof(NearSpace) * r->neuronGroups.size()) : 0);
    r->fusedStage = r->fusedSmemBytes <= 200 * 1024;
    {
        // SPLIT schedule: the warp-specialised kernel, if the neuron slots (dealt out evenly over one
        // CTA per SM) leave at least four warps per CTA free for streaming
        r->streamWarps = 0;
        r->slotsPerCta = 0;
        int sms = 0;
        CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, r->device));
        // (a sharded model on the split schedule measured faster on one set of warps: its chain waits
        // for the other GPUs anyway, and the stream warps' fences compete with it)
        const bool wanted = r->streamWarpsWanted > 0 ||
                            (r->streamWarpsWanted < 0 && !(r->sharded() && r->schedule == b200_runner::SPLIT));
        if((r->schedule == b200_runner::SPLIT || r->schedule == b200_runner::EMIT) && r->fusedStage && wanted && sms > 0) {
            const unsigned int perCta = ((slotStart.back() + sms - 1) / sms + 31u) & ~31u;
            const unsigned int warps = FUSED_BLOCK / 32;
            const unsigned int chainMin = std::max(8u, perCta / 32u);
            // (a sharded model keeps the block's last warp for publishing its spike counts)
            const unsigned int publisher = r->sharded() ? 1u : 0u;
            if(chainMin + 4u + publisher <= warps) {
                unsigned int stream = warps - chainMin - publisher;
                if(r->streamWarpsWanted > 0) stream = std::min(stream, (unsigned int)r->streamWarpsWanted);
                r->streamWarps = stream;
                r->slotsPerCta = perCta;
            }
        }
        if(r->schedule == b200_runner::EMIT && !r->streamWarps) {
            // no room for the warp-specialised kernel after all: plain schedule
            r->schedule = b200_runner::PLAIN;
            return buildFusedTables(r);
        }
        int e = withNeuronShape(r, [&](auto P, auto C) -> int {
            auto fused = fusedStepKernel<decltype(P)::value, decltype(C)::value>;
            auto stream = r->sharded() ? streamStepKernel<decltype(P)::value, decltype(C)::value, true>
                                       : streamStepKernel<decltype(P)::value, decltype(C)::value, false>;
            auto kernel = r->streamWarps ? stream : fused;
            r->fusedKernel = (const void*)kernel;
            if(r->fusedStage) {
                CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)r->fusedSmemBytes));
            }
            int perSM = 0;
            CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSM, kernel, FUSED_BLOCK,
                                                                   r->fusedStage ? r->fusedSmemBytes : 0));
            r->fusedPerSM = perSM;
            return B200_OK;
        });
        if(e) return e;
    }
    CUDA_TRY(cudaMalloc(&r->fusedSlotStart, sizeof(unsigned int) * slotStart.size()));
    CUDA_TRY(cudaMemcpy(r->fusedSlotStart, slotStart.data(), sizeof(unsigned int) * slotStart.size(), cudaMemcpyHostToDevice));
    if(!sources.empty()) {
        CUDA_TRY(cudaMalloc(&r->fusedSources, sizeof(FusedSource) * sources.size()));
        CUDA_TRY(cudaMemcpy(r->fusedSources, sources.data(), sizeof(FusedSource) * sources.size(), cudaMemcpyHostToDevice));
        CUDA_TRY(cudaMalloc(&r->fusedItems, sizeof(uint2) * items.size()));
        CUDA_TRY(cudaMemcpy(r->fusedItems, items.data(), sizeof(uint2) * items.size(), cudaMemcpyHostToDevice));
    }
    if(!r->fusedBarrier) CUDA_TRY(cudaMalloc(&r->fusedBarrier, sizeof(unsigned long long)));
    int perSM = r->fusedPerSM, sms = 0, coop = 0;
    CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, r->device));
    CUDA_TRY(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, r->device));
    if(perSM < 1 || !coop) {
        r->fusedEligible = false;
    }
    else {
        if(r->fusedBlocksPerSM) perSM = std::min<int>(perSM, (int)r->fusedBlocksPerSM);
        if(r->streamWarps) perSM = 1;       // its neuron slots were dealt out for one CTA per SM
        r->fusedGrid = (unsigned int)(perSM * sms);
    }
    return B200_OK;
}

int prepare(b200_runner *r)
{
    if(!r->dirty) return B200_OK;
    r->dropGraph();
    // neuron groups: padded to whole blocks
    {
        std::vector<unsigned int> starts{0};
        for(const auto &g : r->neuronGroups) {
            starts.push_back(starts.back() + (g.num_update + NEURON_BLOCK - 1) / NEURON_BLOCK);
        }
        CUDA_TRY(r->neuronTable.upload(r->neuronGroups, starts, r->stream));
    }
    std::vector<b200_synapse_group> sparse, postSpan, learn, procedural;
    std::vector<unsigned int> sparseStarts{0}, postSpanStarts{0}, learnStarts{0}, proceduralStarts{0};
    for(const auto &g : r->synapseGroups) {
        if(g.connectivity == B200_CONN_SPARSE) {
            sparse.push_back(g);
            // +3: tiles are aligned to the array, not to the row
            sparseStarts.push_back(sparseStarts.back() + (g.row_stride + 3 + PRE_TILE - 1) / PRE_TILE);
        }
        else if(g.connectivity == B200_CONN_BITMASK || g.connectivity == B200_CONN_DENSE) {
            postSpan.push_back(g);
            postSpanStarts.push_back(postSpanStarts.back() + (g.row_stride + PRE_BLOCK - 1) / PRE_BLOCK);
        }
        else if(g.connectivity == B200_CONN_PROCEDURAL) {
            const unsigned int T = connectSubRows(g.proc_connect, g.proc_connect_params);
            if(T > 32u || (T & (T - 1u))) return fail(B200_ERR_INVALID, "procedural group: %u sub-rows per row (a power of two of at most 32 is supported)", T);
            procedural.push_back(g);
            proceduralStarts.push_back(proceduralStarts.back() + 1);
        }
        else {
            return fail(B200_ERR_INVALID, "connectivity %u is not supported by this build", g.connectivity);
        }
        if(g.wu_model == B200_WU_STDP) {
            learn.push_back(g);
            const unsigned int width = (g.connectivity == B200_CONN_SPARSE) ? g.col_stride : g.num_src;
            learnStarts.push_back(learnStarts.back() + (width + POST_BLOCK - 1) / POST_BLOCK);
        }
    }
    CUDA_TRY(r->sparseTable.upload(sparse, sparseStarts, r->stream));
    CUDA_TRY(r->postSpanTable.upload(postSpan, postSpanStarts, r->stream));
    CUDA_TRY(r->learnTable.upload(learn, learnStarts, r->stream));
    CUDA_TRY(r->proceduralTable.upload(procedural, proceduralStarts, r->stream));

    // ---- tables of the persistent fused-step kernel --------------------------------
    r->fusedEligible = (r->batch == 1 && postSpan.empty() && learn.empty() && procedural.empty() &&
                        !r->neuronGroups.empty());
    r->fusedGroups = sparse;
    r->lagStale = true;
    r->tiledStale = true;
    r->schedule = b200_runner::PLAIN;
    r->dropUrgent();
    {
        const int e = buildFusedTables(r);
        if(e) return e;
    }

    // ---- ring period: least common multiple of every ring size ----------------------
    {
        unsigned long long period = 1;
        auto fold = [&period](unsigned int n) {
            if(n < 2) return;
            unsigned long long a = period, b = n;
            while(b) { const unsigned long long t = a % b; a = b; b = t; }
            period = period / a * n;
        };
        for(const auto &g : r->neuronGroups) {
            fold(g.num_delay_slots);
            for(unsigned int p = 0; p < g.num_psm; p++) fold(g.psm[p].max_den_delay);
        }
        for(const auto &g : r->synapseGroups) {
            fold(g.src_delay_slots);
            fold(g.trg_delay_slots);
            fold(g.max_den_delay);
        }
        if(period > (1ull << 30)) return fail(B200_ERR_INVALID, "ring sizes have no common period below 2^30");
        CUDA_TRY(cudaStreamSynchronize(r->stream));
        const unsigned int ring[2] = {(unsigned int)(r->hostStepsDone % period), (unsigned int)period};
        CUDA_TRY(cudaMemcpy(&r->state->phase, ring, sizeof(ring), cudaMemcpyHostToDevice));
    }
    r->dirty = false;
    return B200_OK;
}


// Near-synapse table of the "deliver at emission" schedule; leaves r->schedule alone if the model
// does not qualify (a group without a delay ring of three slots or more, an axonal delay, a ring
// that is not a postsynaptic model of a neuron group, too few free warps for streaming).
int buildNearTables(b200_runner *r, bool forExport = false)
{
    const auto &groups = r->fusedGroups;
    const size_t n = groups.size(), numNeuronGroups = r->neuronGroups.size();
    if(n == 0) return B200_OK;
    unsigned int slots = 0;
    for(const auto &g : r->neuronGroups) slots += (g.num_update + 31u) & ~31u;
    int sms = 0;
    CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, r->device));
    const unsigned int perCta = ((slots + sms - 1) / sms + 31u) & ~31u;
    if(std::max(8u, perCta / 32u) + 4u > FUSED_BLOCK / 32) return B200_OK;      // no room for stream warps
    std::vector<NearRing> rings;
    std::vector<unsigned int> ringOf(n), sourceOf(n);
    for(size_t gi = 0; gi < n; gi++) {
        const auto &g = groups[gi];
        // the stream reads a spike list up to two steps after it was written: delay 0 and four slots
        if(g.max_den_delay < 3 || !g.d || g.axonal_delay != 0 || g.src_delay_slots < 4 || g.num_src >= (1u << 24)) return B200_OK;
        bool found = false;
        for(size_t ni = 0; ni < numNeuronGroups && !found; ni++) {
            const auto &ng = r->neuronGroups[ni];
            for(unsigned int p = 0; p < ng.num_psm && !found; p++) {
                if(ng.psm[p].den_delay == g.den_delay && ng.psm[p].max_den_delay == g.max_den_delay &&
                   ng.num_neurons == g.num_trg) {
                    size_t ri = 0;
                    for(; ri < rings.size(); ri++) if(rings[ri].den_delay == g.den_delay) break;
                    if(ri == rings.size()) rings.push_back(NearRing{g.den_delay, g.max_den_delay, g.num_trg});
                    ringOf[gi] = (unsigned int)ri;
                    found = true;
                }
            }
        }
        if(!found || rings.size() > NEAR_MAX_RINGS) return B200_OK;
        if(forExport) {
            // the other processes reduce into this ring over NVLink: it has to lie in the exchange arena
            const unsigned char *ring = reinterpret_cast<const unsigned char*>(g.den_delay);
            if(ring < r->arena || ring >= r->arena + r->arenaBytes) return B200_OK;
        }
        found = false;
        for(size_t ni = 0; ni < numNeuronGroups && !found; ni++) {
            const auto &ng = r->neuronGroups[ni];
            // the spiking thread looks its row up by neuron id.  One process: it updates the whole
            // population.  Sharded: the rows are built for all source neurons here and handed to
            // the processes that own them (b200_near_import); this process's own list section
            // is `rank` sections into the population's lists.
            const unsigned int *own = g.src_spk_cnt + (forExport ? (size_t)r->rank * g.src_cnt_section_stride : 0);
            if(ng.spk_cnt == own && ng.num_neurons == g.num_src &&
               (forExport || (ng.first_neuron == 0 && ng.num_update == ng.num_neurons))) {
                sourceOf[gi] = (unsigned int)ni;
                found = true;
            }
        }
        if(!found) return B200_OK;
    }
    // rows of every source population, counted first: the longest fixes the population's row length
    std::vector<unsigned long long> rowBase(numNeuronGroups + 1, 0);
    for(size_t ni = 0; ni < numNeuronGroups; ni++) rowBase[ni + 1] = rowBase[ni] + r->neuronGroups[ni].num_neurons;
    const unsigned long long totalRows = rowBase[numNeuronGroups];
    if(totalRows == 0 || totalRows >= (1ull << 31)) return B200_OK;
    // (both freed on every way out of this function; a table left behind by a failed build is dropped with the
    // runner's other near tables)
    ScopedDevice cursorHold, badHold;
    CUDA_TRY(cudaMalloc(&cursorHold.p, sizeof(unsigned int) * totalRows));
    unsigned int *const cursor = cursorHold.as<unsigned int>();
    CUDA_TRY(cudaMemsetAsync(cursor, 0, sizeof(unsigned int) * totalRows, r->stream));
    for(size_t gi = 0; gi < n; gi++) {
        const auto &g = groups[gi];
        if(!g.num_src) continue;
        nearCountKernel<<<std::min(1184u, (g.num_src + 7u) / 8u), 256, 0, r->stream>>>(g, cursor + rowBase[sourceOf[gi]]);
        CUDA_TRY(cudaPeekAtLastError());
        r->launches++;
    }
    std::vector<unsigned int> counts(totalRows);
    CUDA_TRY(cudaMemcpyAsync(counts.data(), cursor, sizeof(unsigned int) * totalRows, cudaMemcpyDeviceToHost, r->stream));
    CUDA_TRY(cudaStreamSynchronize(r->stream));
    std::vector<unsigned long long> firstCell(numNeuronGroups, 0ull);
    std::vector<unsigned int> shifts(numNeuronGroups, 0xFFFFFFFFu);
    unsigned long long cells = 0;
    for(size_t ni = 0; ni < numNeuronGroups; ni++) {
        bool isSource = false;
        for(size_t gi = 0; gi < n; gi++) isSource = isSource || sourceOf[gi] == ni;
        if(!isSource) continue;
        unsigned int longest = 0;
        for(unsigned long long row = rowBase[ni]; row < rowBase[ni + 1]; row++) longest = std::max(longest, counts[row]);
        unsigned int shift = 5;
        while((1u << shift) < longest) shift++;
        // a population most of whose synapses are near gains nothing from this schedule
        if(shift > 10) return B200_OK;
        firstCell[ni] = cells;
        shifts[ni] = shift;
        cells += (unsigned long long)r->neuronGroups[ni].num_neurons << shift;
    }
    if(cells >= (1ull << 33)) return B200_OK;      // 64 GB of table: not worth it
    CUDA_TRY(cudaMemsetAsync(cursor, 0, sizeof(unsigned int) * totalRows, r->stream));
    CUDA_TRY(cudaMalloc(&badHold.p, sizeof(unsigned int)));
    unsigned int *const bad = badHold.as<unsigned int>();
    CUDA_TRY(cudaMemsetAsync(bad, 0, sizeof(unsigned int), r->stream));
    CUDA_TRY(cudaMalloc(&r->nearTable, sizeof(uint2) * (cells + 1)));
    CUDA_TRY(cudaMemsetAsync(r->nearTable, 0, sizeof(uint2) * (cells + 1), r->stream));
    for(size_t gi = 0; gi < n; gi++) {
        const auto &g = groups[gi];
        if(!g.num_src) continue;
        const unsigned int blocks = std::min(1184u, (g.num_src + 7u) / 8u);
        const unsigned int src = sourceOf[gi];
        const int e = withIndType(g.ind_bytes, [&](auto tag) -> int {
            using IndT = decltype(tag);
            nearFillKernel<IndT><<<blocks, 256, 0, r->stream>>>(g, ringOf[gi], cursor + rowBase[src],
                                                                r->nearTable + firstCell[src], shifts[src], bad);
            return B200_OK;
        });
        if(e) return e;
        CUDA_TRY(cudaPeekAtLastError());
        r->launches++;
    }
    unsigned int isBad = 0;
    CUDA_TRY(cudaMemcpyAsync(&isBad, bad, sizeof(unsigned int), cudaMemcpyDeviceToHost, r->stream));
    CUDA_TRY(cudaStreamSynchronize(r->stream));
    if(isBad) {
        cudaFree(r->nearTable);
        r->nearTable = nullptr;
        return B200_OK;
    }
    r->numRings = (unsigned int)rings.size();
    r->nearRingsHost = rings;
    r->nearCellHost = firstCell;
    r->nearShiftHost = shifts;
    if(forExport) return B200_OK;       // the owners of the source neurons take their rows from here
    std::vector<NearSpace> spaces(numNeuronGroups);
    for(size_t ni = 0; ni < numNeuronGroups; ni++) spaces[ni] = NearSpace{r->nearTable + firstCell[ni], shifts[ni], 0u, shifts[ni], 0u};
    CUDA_TRY(cudaMalloc(&r->nearRings, sizeof(NearRing) * rings.size()));
    CUDA_TRY(cudaMemcpy(r->nearRings, rings.data(), sizeof(NearRing) * rings.size(), cudaMemcpyHostToDevice));
    CUDA_TRY(cudaMalloc(&r->nearSpaces, sizeof(NearSpace) * spaces.size()));
    CUDA_TRY(cudaMemcpy(r->nearSpaces, spaces.data(), sizeof(NearSpace) * spaces.size(), cudaMemcpyHostToDevice));
    r->schedule = b200_runner::EMIT;
    return B200_OK;
}

// Choose the schedule of the persistent kernel from the dendritic delays that
// are actually in the arrays, and build what it needs:
//   LAG    every SPARSE group has a delay ring and no synapse arrives in the same
//          step: spikes are delivered one step late, one grid barrier per step;
//   SPLIT  the synapses that do arrive in the same step are copied into tables of
//          their own and delivered before the neuron update, all others after it;
//   PLAIN  everything before the neuron update.
int refreshSchedule(b200_runner *r)
{
    r->lagStale = false;
    r->lagEligible = false;
    r->schedule = b200_runner::PLAIN;
    r->dropUrgent();
    if(!r->fusedEligible) return B200_OK;
    const auto &groups = r->fusedGroups;
    const size_t n = groups.size();
    // rows of every group with a delay ring, one after the other, each group with one extra
    // cell so that offsets[row + 1] exists for its last row
    std::vector<size_t> rowBase(n, 0);
    size_t totalRows = 0;
    bool anyRing = false;
    for(size_t gi = 0; gi < n; gi++) {
        const auto &g = groups[gi];
        if(g.max_den_delay < 2 || !g.d || g.num_src == 0) continue;
        anyRing = true;
        rowBase[gi] = totalRows;
        totalRows += (size_t)g.num_src + 1;
    }
    if((r->useLag || r->useSplit) && anyRing && totalRows < (1ull << 31)) {
        CUDA_TRY(cudaMalloc(&r->urgentOffsets, sizeof(unsigned int) * (totalRows + 1)));
        CUDA_TRY(cudaMemsetAsync(r->urgentOffsets, 0, sizeof(unsigned int) * (totalRows + 1), r->stream));
        for(size_t gi = 0; gi < n; gi++) {
            const auto &g = groups[gi];
            if(g.max_den_delay < 2 || !g.d || g.num_src == 0) continue;
            urgentCountKernel<<<std::min(1184u, (g.num_src + 7u) / 8u), 256, 0, r->stream>>>(g, r->urgentOffsets + rowBase[gi]);
            CUDA_TRY(cudaPeekAtLastError());
            r->launches++;
        }
        // counts -> offsets on the host (a few MB once per change of the delay arrays)
        std::vector<unsigned int> cells(totalRows + 1);
        CUDA_TRY(cudaMemcpyAsync(cells.data(), r->urgentOffsets, sizeof(unsigned int) * (totalRows + 1),
                                 cudaMemcpyDeviceToHost, r->stream));
        CUDA_TRY(cudaStreamSynchronize(r->stream));
        r->urgentStride.assign(n, 0u);
        unsigned long long total = 0;
        for(size_t gi = 0; gi < n; gi++) {
            const auto &g = groups[gi];
            if(g.max_den_delay < 2 || !g.d || g.num_src == 0) continue;
            unsigned int longest = 0;
            for(size_t row = 0; row <= g.num_src; row++) {
                unsigned int &cell = cells[rowBase[gi] + row];
                const unsigned int len = (row < g.num_src) ? cell : 0u;
                longest = std::max(longest, len);
                cell = (unsigned int)total;
                total += len;
            }
            r->urgentStride[gi] = longest;
        }
        // a list read one step late, with a peer possibly writing two steps ahead, needs delay + 4 slots
        bool lagOk = (total == 0);
        for(size_t gi = 0; gi < n; gi++) {
            const auto &g = groups[gi];
            if(g.max_den_delay < 2 || !g.d || g.axonal_delay + 4 > g.src_delay_slots) lagOk = false;
        }
        r->lagEligible = lagOk;
        if(r->useLag && lagOk && (!r->sharded() || r->lagAgreed)) {
            r->schedule = b200_runner::LAG;
        }
        else if(r->useEmit && r->sharded() && r->emitAgreed) {
            if(r->nearDataStale) {
                return fail(B200_ERR_STATE, "synapse arrays of a sharded model changed after its processes exchanged "
                                            "their near-synapse tables: run b200_near_export / import / finish again");
            }
            r->schedule = b200_runner::EMIT;        // tables exchanged between the processes beforehand
        }
        else if(r->useEmit && !r->sharded() && r->streamWarpsWanted != 0 && r->fusedStage) {
            const int e = buildNearTables(r);
            if(e) return e;
        }
        if(r->schedule != b200_runner::PLAIN) {
            // decided
        }
        else if(r->useSplit && total < (1ull << 31)) {
            r->schedule = b200_runner::SPLIT;
            if(total) {
                CUDA_TRY(cudaMemcpyAsync(r->urgentOffsets, cells.data(), sizeof(unsigned int) * (totalRows + 1),
                                         cudaMemcpyHostToDevice, r->stream));
                CUDA_TRY(cudaMalloc(&r->urgentEntries, sizeof(uint2) * total));
                std::vector<FusedUrgent> table(n);
                for(size_t gi = 0; gi < n; gi++) {
                    const auto &g = groups[gi];
                    table[gi] = FusedUrgent{r->urgentOffsets + rowBase[gi], r->urgentEntries, r->urgentStride[gi], 0u};
                    if(!r->urgentStride[gi]) continue;
                    const unsigned int blocks = std::min(1184u, (g.num_src + 7u) / 8u);
                    const int e = withIndType(g.ind_bytes, [&](auto tag) -> int {
                        using IndT = decltype(tag);
                        urgentFillKernel<IndT><<<blocks, 256, 0, r->stream>>>(g, r->urgentOffsets + rowBase[gi], r->urgentEntries);
                        return B200_OK;
                    });
                    if(e) return e;
                    CUDA_TRY(cudaPeekAtLastError());
                    r->launches++;
                }
                CUDA_TRY(cudaMalloc(&r->fusedUrgent, sizeof(FusedUrgent) * n));
                CUDA_TRY(cudaMemcpyAsync(r->fusedUrgent, table.data(), sizeof(FusedUrgent) * n, cudaMemcpyHostToDevice, r->stream));
                CUDA_TRY(cudaStreamSynchronize(r->stream));
            }
        }
        if(!r->urgentEntries) {
            cudaFree(r->urgentOffsets);
            r->urgentOffsets = nullptr;
            r->urgentStride.assign(n, 0u);
        }
    }
    return buildFusedTables(r);
}

// true if [p, p + bytes) overlaps an array the delay scan depends on
bool touchesDelays(const b200_runner *r, const void *p, size_t bytes)
{
    const unsigned char *a = static_cast<const unsigned char*>(p), *b = a + bytes;
    auto overlaps = [&](const void *start, size_t size) {
        const unsigned char *s0 = static_cast<const unsigned char*>(start);
        return s0 && a < s0 + size && b > s0;
    };
    for(const auto &g : r->fusedGroups) {
        if(!g.max_den_delay || !g.d) continue;
        const size_t synapses = (size_t)g.num_src * g.row_stride;
        // the urgent tables copy indices and weights, the schedule depends on delays and row lengths
        if(overlaps(g.d, synapses) || overlaps(g.row_length, sizeof(unsigned int) * g.num_src) ||
           overlaps(g.ind, synapses * g.ind_bytes) || overlaps(g.g, synapses * sizeof(float))) return true;
    }
    return false;
}

// true if [p, p + bytes) overlaps an array the tile-major copy of the SPARSE groups was made from
bool touchesSparse(const b200_runner *r, const void *p, size_t bytes)
{
    const unsigned char *a = static_cast<const unsigned char*>(p), *b = a + bytes;
    auto overlaps = [&](const void *start, size_t size) {
        const unsigned char *s0 = static_cast<const unsigned char*>(start);
        return s0 && a < s0 + size && b > s0;
    };
    for(const auto &g : r->synapseGroups) {
        if(g.connectivity != B200_CONN_SPARSE || g.wu_model == B200_WU_STDP) continue;
        const size_t synapses = (size_t)g.num_src * g.row_stride;
        if(overlaps(g.d, synapses) || overlaps(g.row_length, sizeof(unsigned int) * g.num_src) ||
           overlaps(g.ind, synapses * g.ind_bytes) || overlaps(g.g, synapses * sizeof(float))) return true;
    }
    return false;
}

int launchFused(b200_runner *r, unsigned long long numSteps, unsigned long long numRec)
{
    if(r->lagStale) {
        const bool was = r->lagEligible;
        const int e = refreshSchedule(r);
        if(e) return e;
        if(r->sharded() && r->lagAgreed && r->useLag && was && !r->lagEligible) {
            return fail(B200_ERR_STATE, "a synapse with dendritic delay 0 appeared after the processes of this sharded "
                                        "model agreed to deliver spikes one step late");
        }
    }
    FusedLaunch L;
    L.lag = (r->schedule == b200_runner::LAG) ? 1u : 0u;
    L.skip_urgent = (r->schedule == b200_runner::SPLIT) ? 1u : 0u;
    L.urgent = r->fusedUrgent;
    L.stream_warps = r->streamWarps;
    L.slots_per_cta = r->slotsPerCta;
    L.emit = (r->schedule == b200_runner::EMIT) ? 1u : 0u;
    L.num_rings = r->numRings;
    L.near_rings = r->nearRings;
    L.near_spaces = r->nearSpaces;
    L.queue_words = (r->sharded() && L.emit && r->useNearQueues && r->queuesAgreed) ? r->queueWords : 0u;
    L.queue_count = NEAR_QUEUE_COUNT;
    L.publisher = (r->sharded() && r->streamWarps) ? 1u : 0u;
    L.queue_offset = r->queueOffset;
    L.neuron.groups = r->neuronTable.d;
    L.neuron.block_start = r->neuronTable.blockStart;
    L.neuron.num_groups = r->neuronTable.num;
    L.neuron.batch = 1;
    L.neuron.dt = r->dt;
    L.neuron.seed = r->seed;
    L.neuron.num_recording_timesteps = numRec;
    L.neuron.state = r->state;
    L.neuron.count_events = r->countEvents ? 1u : 0u;
    L.slot_start = r->fusedSlotStart;
    L.sgroups = r->sparseTable.d;
    L.sources = r->fusedSources;
    L.items = r->fusedItems;
    L.num_sources = r->fusedNumSources;
    L.num_sgroups = r->sparseTable.num;
    L.num_items = r->fusedNumItems;
    L.stage_in_smem = r->fusedStage ? 1u : 0u;
    L.count_events = r->countEvents ? 1u : 0u;
    L.profile = r->fusedProfile ? 1u : 0u;
    L.cta_cycles = (r->fusedProfile && r->fusedGrid <= PROFILE_MAX_CTAS) ? r->fusedCtaCycles : nullptr;
    L.num_steps = numSteps;
    L.barrier = r->fusedBarrier;
    L.rank = r->rank;
    L.world = r->world;
    L.arena = r->arena;
    L.peer_table = r->peerTable;
    if(r->sharded()) {
        for(unsigned int p = 0; p < r->world; p++) {
            if(p != r->rank && !r->peerArena[p]) return fail(B200_ERR_STATE, "exchange arena of rank %u has not been opened", p);
        }
        for(const auto &g : r->neuronGroups) {
            const unsigned char *c = reinterpret_cast<const unsigned char*>(g.spk_cnt), *s = reinterpret_cast<const unsigned char*>(g.spk);
            const unsigned char *t = reinterpret_cast<const unsigned char*>(g.spk_tag);
            const unsigned char *w = reinterpret_cast<const unsigned char*>(g.spk_wire);
            if(c < r->arena || c >= r->arena + r->arenaBytes || s < r->arena || s >= r->arena + r->arenaBytes ||
               t < r->arena || t >= r->arena + r->arenaBytes || w < r->arena || w >= r->arena + r->arenaBytes) {
                return fail(B200_ERR_INVALID, "spike arrays of a sharded model must live in the exchange arena");
            }
        }
    }
    CUDA_TRY(cudaMemsetAsync(r->fusedBarrier, 0, sizeof(unsigned long long), r->stream));
    void *args[] = {&L};
    CUDA_TRY(cudaLaunchCooperativeKernel(r->fusedKernel, dim3(r->fusedGrid), dim3(FUSED_BLOCK), args,
                                         r->fusedStage ? r->fusedSmemBytes : 0, r->stream));
    r->launches++;
    r->fusedLaunches++;
    return B200_OK;
}

SynapseLaunch synapseLaunch(const b200_runner *r, const DeviceTable<b200_synapse_group> &t)
{
    SynapseLaunch L;
    L.groups = t.d;
    L.block_start = t.blockStart;
    L.num_groups = t.num;
    L.batch = r->batch;
    L.dt = r->dt;
    L.seed = r->seed;
    L.state = r->state;
    L.count_events = r->countEvents ? 1u : 0u;
    L.tiled_served = nullptr;
    return L;
}

struct ScopedTimer
{
    b200_runner *r;
    std::string name;
    bool on;
    ScopedTimer(b200_runner *r_, const std::string &n, bool capturing) : r(r_), name(n), on(r_->timing && !capturing)
    {
        if(on) cudaEventRecord(r->evA, r->stream);
    }
    ~ScopedTimer()
    {
        if(on) {
            cudaEventRecord(r->evB, r->stream);
            cudaEventSynchronize(r->evB);
            float ms = 0.0f;
            cudaEventElapsedTime(&ms, r->evA, r->evB);
            r->timers[name].seconds += ms * 1e-3;
        }
    }
};

using TiledKernel = void (*)(const TiledLaunch);
TiledKernel tiledKernelFor(bool key16, bool weights)
{
    if(key16) return weights ? tiledDeliverKernel<uint16_t, true> : tiledDeliverKernel<uint16_t, false>;
    return weights ? tiledDeliverKernel<uint32_t, true> : tiledDeliverKernel<uint32_t, false>;
}

// (Re)build the private tile-major copy of the non-learning SPARSE groups (tiled.cuh).  Not on the
// time-step path: runs when the per-kernel path is first used and after the arrays it copies changed.
int buildTiled(b200_runner *r)
{
    r->dropTiled();
    r->tiledStale = false;
    r->tiledWhyNot.clear();
    if(!r->useTiled) { r->tiledWhyNot = "switched off"; return B200_OK; }
    if(r->sharded()) { r->tiledWhyNot = "sharded models run on the persistent kernel"; return B200_OK; }
    // the SPARSE groups in the order of sparseTable; the non-learning ones are served
    std::vector<b200_synapse_group> sparse;
    for(const auto &g : r->synapseGroups) if(g.connectivity == B200_CONN_SPARSE) sparse.push_back(g);
    std::vector<unsigned char> served(sparse.size(), 0);
    struct Target { float *ptr; unsigned int n, depth, stride, tiles, firstTile, firstTable, rows, firstSource; std::vector<size_t> groups; };
    std::vector<Target> targets;
    unsigned int maxDepth = 1;
    unsigned long long slots = 0;
    bool anyWeights = false;
    for(size_t i = 0; i < sparse.size(); i++) {
        const auto &g = sparse[i];
        if(g.wu_model == B200_WU_STDP || g.src_sections > 1) continue;
        float *ptr = g.max_den_delay ? g.den_delay : g.out_post;
        const unsigned int depth = std::max(1u, g.max_den_delay);
        auto it = std::find_if(targets.begin(), targets.end(), [&](const Target &t) { return t.ptr == ptr; });
        if(it == targets.end()) {
            targets.push_back(Target{ptr, g.num_trg, depth, 0, 0, 0, 0, 0, 0, {}});
            it = targets.end() - 1;
        }
        if(it->n != g.num_trg || it->depth != depth) { r->tiledWhyNot = "groups disagree on the shape of a shared target"; return B200_OK; }
        it->groups.push_back(i);
        served[i] = 1;
        maxDepth = std::max(maxDepth, depth);
        slots += (unsigned long long)g.num_src * g.row_stride;
        anyWeights = anyWeights || (g.g != nullptr && g.wu_model != B200_WU_STATIC_PULSE_CONSTANT_WEIGHT);
    }
    if(targets.empty()) { r->tiledWhyNot = "no non-learning SPARSE group"; return B200_OK; }
    for(const auto &t : targets) {
        if(t.groups.size() > TILED_MAX_SOURCES) { r->tiledWhyNot = "too many synapse groups onto one target"; return B200_OK; }
    }
    if(slots >= (1ull << 32)) { r->tiledWhyNot = "more than 2^32 synapse slots"; return B200_OK; }
    if(maxDepth > TILED_ACC_FLOATS || maxDepth > 4096u) { r->tiledWhyNot = "delay ring too deep for a shared-memory tile"; return B200_OK; }
    const bool key16 = (maxDepth <= 64u);
    const unsigned int postBits = key16 ? 10u : 20u;
    unsigned int numTiles = 0, entries = 0, numSources = 0;
    for(auto &t : targets) {
        t.stride = std::min(std::min(1u << postBits, TILED_ACC_FLOATS / t.depth), std::max(t.n, 1u));
        t.tiles = (t.n + t.stride - 1) / t.stride;
        t.rows = 1;
        for(size_t gi : t.groups) t.rows += sparse[gi].num_src;
        t.firstTile = numTiles;
        t.firstTable = entries;
        t.firstSource = numSources;
        const unsigned long long e = (unsigned long long)entries + (unsigned long long)t.tiles * t.rows;
        if(e >= (1ull << 32)) { r->tiledWhyNot = "run-start tables exceed 2^32 entries"; return B200_OK; }
        entries = (unsigned int)e;
        numTiles += t.tiles;
        numSources += (unsigned int)t.groups.size();
    }
    if(numTiles > 65535u) { r->tiledWhyNot = "more than 65535 tiles"; return B200_OK; }

    // ---- count, scan, place ---------------------------------------------------------------------
    ScopedDevice count, runStart, scanTemp, keys, weights;
    CUDA_TRY(cudaMalloc(&count.p, sizeof(unsigned int) * ((size_t)entries + 1)));
    CUDA_TRY(cudaMalloc(&runStart.p, sizeof(unsigned int) * ((size_t)entries + 1)));
    CUDA_TRY(cudaMemsetAsync(count.p, 0, sizeof(unsigned int) * ((size_t)entries + 1), r->stream));
    std::vector<TiledBuildGroup> build;
    std::vector<TiledSource> sources;
    for(auto &t : targets) {
        unsigned int rowBase = 0;
        for(size_t gi : t.groups) {
            const auto &g = sparse[gi];
            TiledBuildGroup B{};
            B.row_length = g.row_length; B.ind = g.ind; B.d = g.max_den_delay ? g.d : nullptr;
            B.g = (g.wu_model == B200_WU_STATIC_PULSE_CONSTANT_WEIGHT) ? nullptr : g.g;
            B.num_src = g.num_src; B.row_stride = g.row_stride; B.ind_bytes = g.ind_bytes; B.num_trg = g.num_trg;
            B.depth = t.depth; B.first_tile = t.firstTile; B.stride = t.stride; B.row_base = rowBase;
            B.rows_per_tile = t.rows; B.first_table = t.firstTable; B.const_weight = g.wu_params[0];
            build.push_back(B);
            TiledSource S{};
            S.spk_cnt = g.src_spk_cnt; S.spk = g.src_spk; S.num_src = g.num_src; S.src_delay_slots = g.src_delay_slots;
            S.axonal_delay = g.axonal_delay; S.row_base = rowBase; S.const_weight = g.wu_params[0]; S.mean_row = 0.0f;
            sources.push_back(S);
            rowBase += g.num_src;
        }
    }
    auto launchBuild = [&](int pass) -> int {
        for(const auto &B : build) {
            const unsigned long long total = (unsigned long long)B.num_src * B.row_stride;
            if(!total) continue;
            const unsigned int blocks = (unsigned int)std::min<unsigned long long>((total + 255) / 256, 148ull * 16ull);
            if(key16) tiledBuildKernel<uint16_t><<<blocks, 256, 0, r->stream>>>(B, pass, count.as<unsigned int>(), runStart.as<unsigned int>(),
                                                                            keys.as<uint16_t>(), weights.as<float>(), postBits, r->state);
            else tiledBuildKernel<uint32_t><<<blocks, 256, 0, r->stream>>>(B, pass, count.as<unsigned int>(), runStart.as<unsigned int>(),
                                                                       keys.as<uint32_t>(), weights.as<float>(), postBits, r->state);
            r->launches++;
        }
        CUDA_TRY(cudaPeekAtLastError());
        return B200_OK;
    };
    if(const int e = launchBuild(0)) return e;
    size_t tempBytes = 0;
    CUDA_TRY(cub::DeviceScan::ExclusiveSum(nullptr, tempBytes, count.as<unsigned int>(), runStart.as<unsigned int>(), (int)(entries + 1), r->stream));
    CUDA_TRY(cudaMalloc(&scanTemp.p, std::max<size_t>(tempBytes, 16)));
    CUDA_TRY(cub::DeviceScan::ExclusiveSum(scanTemp.p, tempBytes, count.as<unsigned int>(), runStart.as<unsigned int>(), (int)(entries + 1), r->stream));
    unsigned int total = 0;
    CUDA_TRY(cudaMemcpyAsync(&total, runStart.as<unsigned int>() + entries, sizeof(total), cudaMemcpyDeviceToHost, r->stream));
    CUDA_TRY(cudaStreamSynchronize(r->stream));
    CUDA_TRY(cudaMalloc(&keys.p, std::max<size_t>((size_t)total * (key16 ? 2 : 4), 16)));
    if(anyWeights) CUDA_TRY(cudaMalloc(&weights.p, std::max<size_t>((size_t)total * sizeof(float), 16)));
    CUDA_TRY(cudaMemsetAsync(count.p, 0, sizeof(unsigned int) * ((size_t)entries + 1), r->stream));
    if(const int e = launchBuild(1)) return e;

    // ---- tiles, sources and (tile, source) pairs -----------------------------------------------------
    std::vector<unsigned int> hostRuns((size_t)entries + 1);
    CUDA_TRY(cudaMemcpyAsync(hostRuns.data(), runStart.p, sizeof(unsigned int) * hostRuns.size(), cudaMemcpyDeviceToHost, r->stream));
    CUDA_TRY(cudaStreamSynchronize(r->stream));
    std::vector<TiledTile> tiles(numTiles);
    std::vector<TiledPair> pairs;
    {
        size_t firstSource = 0;
        for(auto &t : targets) {
            std::vector<unsigned long long> groupSynapses(t.groups.size(), 0);
            for(unsigned int i = 0; i < t.tiles; i++) {
                TiledTile &T = tiles[t.firstTile + i];
                T.target = t.ptr; T.num_trg = t.n; T.depth = t.depth; T.first_trg = i * t.stride;
                T.num_tile = std::min(t.stride, t.n - i * t.stride); T.stride = t.stride;
                T.first_source = t.firstSource; T.num_sources = (unsigned int)t.groups.size();
                T.table = t.firstTable + i * t.rows;
                for(size_t si = 0; si < t.groups.size(); si++) {
                    const auto &g = sparse[t.groups[si]];
                    const size_t base = (size_t)T.table + sources[firstSource + si].row_base;
                    const unsigned long long syn = hostRuns[base + g.num_src] - hostRuns[base];
                    groupSynapses[si] += syn;
                    if(syn) {
                        pairs.push_back(TiledPair{(unsigned short)(t.firstTile + i), (unsigned short)si,
                                                  (float)((double)syn / std::max(1u, g.num_src))});
                    }
                }
            }
            // per source: synapses per source neuron, for the event estimate of a step
            for(size_t si = 0; si < t.groups.size(); si++) {
                const auto &g = sparse[t.groups[si]];
                sources[firstSource + si].mean_row = g.num_src ? (float)((double)groupSynapses[si] / g.num_src) : 0.0f;
            }
            firstSource += t.groups.size();
        }
    }
    if(pairs.empty()) { r->tiledWhyNot = "no synapses"; return B200_OK; }
    if((unsigned long long)pairs.size() * r->batch >= (1ull << 31)) { r->tiledWhyNot = "too many (tile, source, batch) pairs"; return B200_OK; }
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, r->device));
    const unsigned int grid = (unsigned int)prop.multiProcessorCount;
    size_t smem = 0;
    for(const auto &T : tiles) smem = std::max(smem, sizeof(float) * T.depth * T.stride);
    auto toDevice = [&](const void *host, size_t bytes, void **out) -> int {
        CUDA_TRY(cudaMalloc(out, std::max<size_t>(bytes, 16)));
        CUDA_TRY(cudaMemcpy(*out, host, bytes, cudaMemcpyHostToDevice));
        return B200_OK;
    };
    int e = toDevice(tiles.data(), sizeof(TiledTile) * tiles.size(), (void**)&r->tiledTiles);
    if(!e) e = toDevice(sources.data(), sizeof(TiledSource) * sources.size(), (void**)&r->tiledSources);
    if(!e) e = toDevice(pairs.data(), sizeof(TiledPair) * pairs.size(), (void**)&r->tiledPairs);
    if(!e) e = toDevice(served.data(), served.size(), (void**)&r->tiledServed);
    if(e) { r->dropTiled(); return e; }
    // scratch of the per-step work partition
    {
        const size_t perStep = pairs.size() * r->batch;
        cudaError_t ce = cudaMalloc(&r->tiledPairBatches, sizeof(unsigned int) * perStep);
        if(ce == cudaSuccess) ce = cudaMalloc(&r->tiledPairPrefix, sizeof(double) * perStep);
        if(ce == cudaSuccess) ce = cudaMalloc(&r->tiledCtaStart, sizeof(unsigned int) * 2 * (grid + 1));
        if(ce != cudaSuccess) { r->dropTiled(); CUDA_TRY(ce); }
    }
    CUDA_TRY(cudaFuncSetAttribute(tiledKernelFor(key16, anyWeights), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    r->tiledRunStart = static_cast<unsigned int*>(runStart.release());
    r->tiledKeys = keys.release();
    r->tiledWeights = static_cast<float*>(weights.release());
    r->tiledNumPairs = (unsigned int)pairs.size();
    r->tiledNumSources = numSources;
    r->tiledPostBits = postBits;
    r->tiledGrid = grid;
    r->tiledSmemBytes = smem;
    r->tiledSynapses = total;
    if(!r->peakHost) {
        // where the neuron kernel's spike-count peaks land (allocated here, with the copy; never on the time-step path)
        CUDA_TRY(cudaHostAlloc(reinterpret_cast<void**>(&r->peakHost), sizeof(unsigned int), cudaHostAllocPortable));
        CUDA_TRY(cudaEventCreateWithFlags(&r->peakEvent, cudaEventDisableTiming));
        *r->peakHost = 0u;
    }
    r->tiledReady = true;
    {
        unsigned long long neurons = 0;
        for(const auto &ng : r->neuronGroups) neurons += ng.num_neurons;
        r->eventsPerSpike = neurons ? (double)r->tiledSynapses / (double)neurons : 0.0;
    }
    return B200_OK;
}

TiledLaunch tiledLaunch(const b200_runner *r)
{
    TiledLaunch L;
    L.tiles = r->tiledTiles; L.sources = r->tiledSources; L.run_start = r->tiledRunStart; L.keys = r->tiledKeys;
    L.weights = r->tiledWeights; L.pairs = r->tiledPairs; L.pair_batches = r->tiledPairBatches;
    L.pair_prefix = r->tiledPairPrefix; L.cta_start = r->tiledCtaStart; L.num_pairs = r->tiledNumPairs;
    L.num_sources = r->tiledNumSources; L.grid = r->tiledGrid;
    L.batch = r->batch; L.post_bits = r->tiledPostBits; L.min_events = r->tiledMinEvents; L.state = r->state;
    L.count_events = r->countEvents ? 1u : 0u;
    L.ticket_events = r->tiledTicketEvents; L.ticket_cost = r->tiledTicketCost;
    L.profile = (r->fusedProfile && r->tiledGrid <= PROFILE_MAX_CTAS) ? r->fusedCtaCycles : nullptr;
    return L;
}

// Before steps are enqueued (or captured) on the one-launch-per-kernel path.
int ensureTiled(b200_runner *r)
{
    if(r->sparseTable.num && (r->tiledStale || (r->useTiled && !r->tiledReady && r->tiledWhyNot.empty()))) {
        r->dropGraph();
        return buildTiled(r);
    }
    return B200_OK;
}

// (`force`: an update the caller asked for on its own, with spike lists of its choosing)
bool tiledActive(const b200_runner *r, bool force = false)
{
    return r->tiledReady && (force || r->tiledArmed || r->tiledMinEvents == 0);
}

int enqueueSynapses(b200_runner *r, bool capturing, bool force = false)
{
    if(r->sparseTable.num) {
        ScopedTimer tm(r, "presynaptic_update", capturing);
        SynapseLaunch S = synapseLaunch(r, r->sparseTable);
        if(tiledActive(r, force)) {
            // the step's estimated events decide which of the two kernels delivers the served groups
            const TiledLaunch T = tiledLaunch(r);
            tiledDecideKernel<<<1, TILED_BLOCK, 0, r->stream>>>(T);
            tiledKernelFor(r->tiledPostBits == 10u, r->tiledWeights != nullptr)<<<r->tiledGrid, TILED_BLOCK, r->tiledSmemBytes, r->stream>>>(T);
            r->launches += 2;
            S.tiled_served = r->tiledServed;
        }
        const dim3 grid(r->sparseTable.blocks, r->spikeLanes, r->batch);
        presynapticSparseKernel<<<grid, PRE_BLOCK, 0, r->stream>>>(S);
        r->launches++;
    }
    if(r->postSpanTable.num) {
        ScopedTimer tm(r, "presynaptic_update", capturing);
        const dim3 grid(r->postSpanTable.blocks, 1, r->batch);
        presynapticPostSpanKernel<<<grid, PRE_BLOCK, 0, r->stream>>>(synapseLaunch(r, r->postSpanTable));
        r->launches++;
    }
    if(r->proceduralTable.num) {
        ScopedTimer tm(r, "presynaptic_update", capturing);
        // (spike, sub-row) items spread over the whole device; the spike count is only known there
        int sms = 0;
        CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, r->device));
        const dim3 grid((unsigned int)sms * 8u, r->proceduralTable.num, r->batch);
        presynapticProceduralKernel<<<grid, PROC_BLOCK, 0, r->stream>>>(synapseLaunch(r, r->proceduralTable));
        r->launches++;
    }
    if(r->learnTable.num) {
        ScopedTimer tm(r, "postsynaptic_update", capturing);
        const dim3 grid(r->learnTable.blocks, r->spikeLanes, r->batch);
        postsynapticUpdateKernel<<<grid, POST_BLOCK, 0, r->stream>>>(synapseLaunch(r, r->learnTable));
        r->launches++;
    }
    CUDA_TRY(cudaPeekAtLastError());
    return B200_OK;
}

int enqueueNeurons(b200_runner *r, unsigned long long numRec, bool capturing)
{
    if(r->neuronTable.num == 0) return fail(B200_ERR_STATE, "no neuron groups registered");
    ScopedTimer tm(r, "neuron_update", capturing);
    NeuronLaunch L;
    L.groups = r->neuronTable.d;
    L.block_start = r->neuronTable.blockStart;
    L.num_groups = r->neuronTable.num;
    L.batch = r->batch;
    L.dt = r->dt;
    L.seed = r->seed;
    L.num_recording_timesteps = numRec;
    L.state = r->state;
    L.count_events = r->countEvents ? 1u : 0u;
    const dim3 grid(r->neuronTable.blocks, r->batch, 1);
    int e = withNeuronShape(r, [&](auto P, auto C) -> int {
        neuronUpdateKernel<decltype(P)::value, decltype(C)::value><<<grid, NEURON_BLOCK, 0, r->stream>>>(L);
        return B200_OK;
    });
    if(e) return e;
    r->launches++;
    CUDA_TRY(cudaPeekAtLastError());
    return B200_OK;
}

// Behind a block of steps of the per-kernel path: the block's largest spike count on its way to the host.
int fetchPeak(b200_runner *r)
{
    if(!r->peakHost || r->peakPending) return B200_OK;      // (an earlier block's copy still under way: keep it)
    CUDA_TRY(cudaMemcpyAsync(r->peakHost, &r->state->peak_spikes, sizeof(unsigned int), cudaMemcpyDeviceToHost, r->stream));
    CUDA_TRY(cudaMemsetAsync(&r->state->peak_spikes, 0, sizeof(unsigned int), r->stream));
    CUDA_TRY(cudaEventRecord(r->peakEvent, r->stream));
    r->peakPending = true;
    return B200_OK;
}

// Before a block of steps: arm or disarm the tiled kernels from the last spike count that has arrived.
int pollPeak(b200_runner *r)
{
    if(!r->tiledReady || !r->peakPending || cudaEventQuery(r->peakEvent) != cudaSuccess) return B200_OK;
    r->peakPending = false;
    const double estimate = (double)*r->peakHost * r->eventsPerSpike;
    const bool was = r->tiledArmed;
    if(estimate * 4.0 >= (double)r->tiledMinEvents) {
        r->tiledArmed = true;
        r->quietBlocks = 0;
    }
    else if(r->tiledArmed && estimate * 16.0 < (double)r->tiledMinEvents && ++r->quietBlocks >= 3) {
        r->tiledArmed = false;
    }
    if(was != r->tiledArmed) r->dropGraph();        // the captured steps launch other kernels now
    return B200_OK;
}

int enqueueStep(b200_runner *r, unsigned long long numRec, bool capturing)
{
    int e = enqueueSynapses(r, capturing);
    if(e) return e;
    return enqueueNeurons(r, numRec, capturing);
}

unsigned int kernelsPerStep(const b200_runner *r)
{
    return 1u + (r->sparseTable.num ? (tiledActive(r) ? 3u : 1u) : 0u) + (r->postSpanTable.num ? 1u : 0u) + (r->learnTable.num ? 1u : 0u) +
           (r->proceduralTable.num ? 1u : 0u);
}

int buildGraph(b200_runner *r, unsigned int len, unsigned long long numRec)
{
    r->dropGraph();
    cudaGraph_t graph = nullptr;
    const unsigned long long before = r->launches;
    CUDA_TRY(cudaStreamBeginCapture(r->stream, cudaStreamCaptureModeThreadLocal));
    int e = B200_OK;
    for(unsigned int i = 0; i < len && e == B200_OK; i++) e = enqueueStep(r, numRec, true);
    cudaError_t ce = cudaStreamEndCapture(r->stream, &graph);
    r->launches = before;       // capture enqueues nothing
    if(e) {
        if(graph) cudaGraphDestroy(graph);
        return e;
    }
    CUDA_TRY(ce);
    ce = cudaGraphInstantiate(&r->graphExec, graph, 0);
    cudaGraphDestroy(graph);
    CUDA_TRY(ce);
    r->graphLen = len;
    r->graphNumRec = numRec;
    return B200_OK;
}
}   // anonymous namespace

extern "C" {

const char *b200_last_error(void)
{
    return g_lastError.c_str();
}

int b200_device_count(int *count)
{
    CUDA_TRY(cudaGetDeviceCount(count));
    return B200_OK;
}

int b200_runner_create(int device, double dt, uint64_t seed, uint32_t batch_size, b200_runner **out)
{
    if(!out || batch_size == 0) return fail(B200_ERR_INVALID, "bad arguments to b200_runner_create");
    CUDA_TRY(cudaSetDevice(device));
    b200_runner *r = new b200_runner();
    r->device = device;
    r->dt = (float)dt;
    r->seed = seed;
    r->batch = batch_size;
    CUDA_TRY(cudaStreamCreateWithFlags(&r->stream, cudaStreamNonBlocking));
    CUDA_TRY(cudaMalloc(&r->state, sizeof(StepState)));
    CUDA_TRY(cudaMemset(r->state, 0, sizeof(StepState)));
    {
        const unsigned long long limits[3] = {BARRIER_SPIN_LIMIT, EXCHANGE_SPIN_LIMIT, (unsigned long long)STREAM_WAIT_CYCLES};
        CUDA_TRY(cudaMemcpy(&r->state->barrier_spin_limit, limits, sizeof(limits), cudaMemcpyHostToDevice));
    }
    CUDA_TRY(cudaEventCreate(&r->evA));
    CUDA_TRY(cudaEventCreate(&r->evB));
    CUDA_TRY(cudaEventCreate(&r->evC));
    CUDA_TRY(cudaEventCreate(&r->evD));
    *out = r;
    return B200_OK;
}

/* ---- NCCL, resolved when first needed: the library that is already in the process (a host application
 *      that bootstraps with torch.distributed has loaded one) or the system's.  The reference's CUDA backend
 *      exports ncclGenerateUniqueID / ncclGetUniqueID / ncclInitCommunicator from the generated library
 *      and emits one ncclAllReduce per reduction target (backends/cuda/backend.cc:219-226, 1360-1389,
 *      backendCUDAHIP.h:240-292); here the targets of a group travel as ONE buffer. ------------------- */
namespace
{
struct NcclId { char internal[128]; };                  // ncclUniqueId
struct NcclApi
{
    void *lib = nullptr;
    int (*getUniqueId)(NcclId*) = nullptr;
    int (*commInitRank)(void**, int, NcclId, int) = nullptr;
    int (*allReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*commDestroy)(void*) = nullptr;
    const char *(*getErrorString)(int) = nullptr;
};
constexpr int NCCL_FLOAT32 = 7, NCCL_SUM = 0, NCCL_MAX = 2;     // ncclDataType_t / ncclRedOp_t values of nccl.h

NcclApi *ncclApi()
{
    static NcclApi api;
    if(api.lib) return &api;
    void *lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if(!lib) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if(!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    if(!lib) return nullptr;
    api.getUniqueId = reinterpret_cast<decltype(api.getUniqueId)>(dlsym(lib, "ncclGetUniqueId"));
    api.commInitRank = reinterpret_cast<decltype(api.commInitRank)>(dlsym(lib, "ncclCommInitRank"));
    api.allReduce = reinterpret_cast<decltype(api.allReduce)>(dlsym(lib, "ncclAllReduce"));
    api.commDestroy = reinterpret_cast<decltype(api.commDestroy)>(dlsym(lib, "ncclCommDestroy"));
    api.getErrorString = reinterpret_cast<decltype(api.getErrorString)>(dlsym(lib, "ncclGetErrorString"));
    if(!api.getUniqueId || !api.commInitRank || !api.allReduce || !api.commDestroy || !api.getErrorString) return nullptr;
    api.lib = lib;
    return &api;
}
}   // namespace

#define NCCL_TRY(api, call) do { const int e_ = (call); if(e_ != 0) return fail(B200_ERR_CUDA, "NCCL: %s (%s)", (api)->getErrorString(e_), #call); } while(0)

int b200_runner_destroy(b200_runner *r)
{
    if(!r) return B200_OK;
    cudaSetDevice(r->device);
    cudaStreamSynchronize(r->stream);
    r->dropGraph();
    r->neuronTable.release();
    r->sparseTable.release();
    r->postSpanTable.release();
    r->proceduralTable.release();
    r->learnTable.release();
    if(r->fusedSlotStart) cudaFree(r->fusedSlotStart);
    if(r->fusedSources) cudaFree(r->fusedSources);
    if(r->fusedItems) cudaFree(r->fusedItems);
    if(r->fusedBarrier) cudaFree(r->fusedBarrier);
    if(r->lagScan) cudaFree(r->lagScan);
    r->dropUrgent();
    r->dropNear();
    if(r->fusedCtaCycles) cudaFree(r->fusedCtaCycles);
    r->dropTiled();
    for(unsigned int p = 0; p < B200_MAX_RANKS; p++) {
        if(r->peerArena[p] && !r->peerLocal[p]) cudaIpcCloseMemHandle(r->peerArena[p]);
    }
    if(r->peakHost) cudaFreeHost(r->peakHost);
    if(r->peakEvent) cudaEventDestroy(r->peakEvent);
    if(r->ncclComm && ncclApi()) ncclApi()->commDestroy(r->ncclComm);
    if(r->reducePacked) cudaFree(r->reducePacked);
    if(r->arena) cudaFree(r->arena);
    if(r->peerTable) cudaFree(r->peerTable);
    for(auto &a : r->arrays) cudaFree(a.first);
    cudaFree(r->state);
    cudaEventDestroy(r->evA);
    cudaEventDestroy(r->evB);
    cudaEventDestroy(r->evC);
    cudaEventDestroy(r->evD);
    cudaStreamDestroy(r->stream);
    delete r;
    return B200_OK;
}

int b200_array_alloc(b200_runner *r, size_t bytes, void **device_ptr)
{
    if(!r || !device_ptr) return fail(B200_ERR_INVALID, "bad arguments to b200_array_alloc");
    CUDA_TRY(cudaSetDevice(r->device));
    void *p = nullptr;
    CUDA_TRY(cudaMalloc(&p, bytes + ARRAY_TAIL_PAD));
    CUDA_TRY(cudaMemsetAsync(p, 0, bytes + ARRAY_TAIL_PAD, r->stream));
    r->arrays[p] = bytes;
    *device_ptr = p;
    return B200_OK;
}

int b200_host_alloc(b200_runner *r, size_t bytes, void **host_ptr)
{
    if(!r || !host_ptr) return fail(B200_ERR_INVALID, "bad arguments to b200_host_alloc");
    CUDA_TRY(cudaSetDevice(r->device));
    CUDA_TRY(cudaHostAlloc(host_ptr, bytes ? bytes : 1, cudaHostAllocPortable));
    return B200_OK;
}

int b200_host_free(b200_runner *r, void *host_ptr)
{
    (void)r;
    CUDA_TRY(cudaFreeHost(host_ptr));
    return B200_OK;
}

// The arena a process allocates: the caller's bytes, then the near-synapse queues of both step parities
// from every process (the same layout in every process: peers address each other's arenas by offset).
static size_t exchangeQueueOffset(size_t bytes) { return (bytes + 255) & ~(size_t)255; }
static size_t exchangeTotalBytes(size_t bytes)
{
    return exchangeQueueOffset(bytes) + (size_t)2 * B200_MAX_RANKS * NEAR_QUEUE_COUNT * NEAR_QUEUE_WORDS * sizeof(unsigned long long)
        + ARRAY_TAIL_PAD;
}

int b200_exchange_alloc(b200_runner *r, size_t bytes, void **device_ptr)
{
    if(!r || !device_ptr || bytes == 0) return fail(B200_ERR_INVALID, "bad arguments to b200_exchange_alloc");
    if(r->arena) return fail(B200_ERR_STATE, "the exchange arena has already been allocated");
    CUDA_TRY(cudaSetDevice(r->device));
    void *p = nullptr;
    const size_t total = exchangeTotalBytes(bytes);
    CUDA_TRY(cudaMalloc(&p, total));
    CUDA_TRY(cudaMemset(p, 0, total));
    r->arena = static_cast<unsigned char*>(p);
    r->arenaBytes = bytes;
    r->queueOffset = exchangeQueueOffset(bytes);
    *device_ptr = p;
    return B200_OK;
}

int b200_exchange_bytes(b200_runner *r, size_t *bytes)
{
    if(!r || !r->arena || !bytes) return fail(B200_ERR_STATE, "no exchange arena");
    *bytes = exchangeTotalBytes(r->arenaBytes);
    return B200_OK;
}

int b200_exchange_get_handle(b200_runner *r, void *handle_64_bytes)
{
    if(!r || !r->arena || !handle_64_bytes) return fail(B200_ERR_STATE, "no exchange arena");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    CUDA_TRY(cudaIpcGetMemHandle(&h, r->arena));
    memcpy(handle_64_bytes, &h, sizeof(h));
    return B200_OK;
}

int b200_exchange_open_peer(b200_runner *r, uint32_t peer_rank, const void *handle_64_bytes)
{
    if(!r || peer_rank >= B200_MAX_RANKS || !handle_64_bytes) return fail(B200_ERR_INVALID, "bad peer rank");
    if(r->peerArena[peer_rank]) return fail(B200_ERR_STATE, "peer %u already opened", peer_rank);
    CUDA_TRY(cudaSetDevice(r->device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle_64_bytes, sizeof(h));
    void *p = nullptr;
    CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    r->peerArena[peer_rank] = static_cast<unsigned char*>(p);
    if(!r->peerTable) CUDA_TRY(cudaMalloc(&r->peerTable, sizeof(unsigned char*) * B200_MAX_RANKS));
    CUDA_TRY(cudaMemcpy(r->peerTable, r->peerArena, sizeof(unsigned char*) * B200_MAX_RANKS, cudaMemcpyHostToDevice));
    return B200_OK;
}

int b200_exchange_set_peer(b200_runner *r, uint32_t peer_rank, void *device_ptr)
{
    if(!r || peer_rank >= B200_MAX_RANKS || !device_ptr) return fail(B200_ERR_INVALID, "bad peer rank or pointer");
    if(r->peerArena[peer_rank]) return fail(B200_ERR_STATE, "peer %u already opened", peer_rank);
    CUDA_TRY(cudaSetDevice(r->device));
    r->peerArena[peer_rank] = static_cast<unsigned char*>(device_ptr);
    if(!r->peerTable) CUDA_TRY(cudaMalloc(&r->peerTable, sizeof(unsigned char*) * B200_MAX_RANKS));
    CUDA_TRY(cudaMemcpy(r->peerTable, r->peerArena, sizeof(unsigned char*) * B200_MAX_RANKS, cudaMemcpyHostToDevice));
    r->peerLocal[peer_rank] = true;
    return B200_OK;
}

/* ---- sharded "deliver at emission": every process builds the near-synapse rows of ALL source neurons
 *      onto its own neurons, then hands each process the rows of that process's neurons ------------- */
int b200_near_export(b200_runner *r, void *handle_64_bytes, uint64_t *meta, uint32_t meta_words)
{
    if(!r || !handle_64_bytes || !meta) return fail(B200_ERR_INVALID, "null argument");
    CUDA_TRY(cudaSetDevice(r->device));
    int e = prepare(r);
    if(e) return e;
    r->emitAgreed = false;
    r->dropNear();
    memset(handle_64_bytes, 0, 64);
    const size_t groups = r->neuronGroups.size();
    if(meta_words < 3 + 2 * groups) return fail(B200_ERR_INVALID, "meta array too short: %zu words needed", 3 + 2 * groups);
    meta[0] = 0; meta[1] = groups; meta[2] = 0;
    if(!r->sharded() || !r->fusedEligible || !r->useEmit || r->streamWarpsWanted == 0 || !r->fusedStage) return B200_OK;
    e = buildNearTables(r, true);
    if(e) return e;
    if(!r->nearTable) return B200_OK;       // does not qualify
    cudaIpcMemHandle_t h;
    CUDA_TRY(cudaIpcGetMemHandle(&h, r->nearTable));
    memcpy(handle_64_bytes, &h, sizeof(h));
    meta[0] = 1; meta[2] = (uint64_t)r->numRings | ((uint64_t)r->fusedGrid << 32);
    for(size_t ni = 0; ni < groups; ni++) {
        meta[3 + 2 * ni] = r->nearCellHost[ni];
        meta[4 + 2 * ni] = r->nearShiftHost[ni];
    }
    r->nearImported.assign(groups, nullptr);
    r->nearSpacesAll.assign(groups, NearSpace{nullptr, 0xFFFFFFFFu, 0u, 0u, 0u});
    r->nearPeerDone.assign(r->world, false);
    r->nearDataStale = false;
    return B200_OK;
}

int b200_near_import(b200_runner *r, uint32_t peer_rank, const void *handle_64_bytes, const uint64_t *meta,
                     const uint32_t *common_shift)
{
    if(!r || !handle_64_bytes || !meta || !common_shift || peer_rank >= r->world) return fail(B200_ERR_INVALID, "bad arguments to b200_near_import");
    const size_t groups = r->neuronGroups.size();
    if(r->nearImported.size() != groups || r->nearPeerDone.size() != r->world) return fail(B200_ERR_STATE, "b200_near_export has to come first");
    if(!meta[0] || meta[1] != groups || (uint32_t)meta[2] != r->numRings) return fail(B200_ERR_STATE, "process %u does not qualify or runs another model", peer_rank);
    r->peerGrid[peer_rank] = (unsigned int)(meta[2] >> 32);
    CUDA_TRY(cudaSetDevice(r->device));
    const uint2 *table = r->nearTable;
    void *mapped = nullptr;
    if(peer_rank != r->rank) {
        cudaIpcMemHandle_t h;
        memcpy(&h, handle_64_bytes, sizeof(h));
        CUDA_TRY(cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess));
        table = static_cast<const uint2*>(mapped);
    }
    unsigned int worldShift = 0;
    while((1u << worldShift) < r->world) worldShift++;
    // Rows of this process's neurons: [neuron][process][1 << common shift] entries, zero padded.  The
    // block of process `peer_rank` is copied out of that process's table, whose rows may be shorter.
    for(size_t ni = 0; ni < groups; ni++) {
        const uint32_t shift = (uint32_t)meta[4 + 2 * ni], common = common_shift[ni];
        if(shift == 0xFFFFFFFFu || common == 0xFFFFFFFFu) continue;
        if(shift > common || common + worldShift > 12) return fail(B200_ERR_INVALID, "bad common row length for neuron group %zu", ni);
        const auto &ng = r->neuronGroups[ni];
        const size_t rowCells = (size_t)1 << (common + worldShift);
        if(!r->nearImported[ni]) {
            CUDA_TRY(cudaMalloc(&r->nearImported[ni], sizeof(uint2) * (rowCells * ng.num_update + 1)));
            CUDA_TRY(cudaMemset(r->nearImported[ni], 0, sizeof(uint2) * (rowCells * ng.num_update + 1)));
            r->nearSpacesAll[ni] = NearSpace{r->nearImported[ni], common + worldShift, ng.first_neuron, common, 0u};
        }
        if(ng.num_update) {
            CUDA_TRY(cudaMemcpy2D(r->nearImported[ni] + ((size_t)peer_rank << common), sizeof(uint2) * rowCells,
                                  table + meta[3 + 2 * ni] + ((size_t)ng.first_neuron << shift), sizeof(uint2) << shift,
                                  sizeof(uint2) << shift, ng.num_update, cudaMemcpyDeviceToDevice));
        }
    }
    CUDA_TRY(cudaDeviceSynchronize());
    if(mapped) CUDA_TRY(cudaIpcCloseMemHandle(mapped));
    r->nearPeerDone[peer_rank] = true;
    return B200_OK;
}

/* After EVERY process has imported from every process (the caller synchronises them): free the full table
 * and switch the schedule on (`agreed` != 0) or drop everything. */
int b200_near_finish(b200_runner *r, int agreed)
{
    if(!r) return fail(B200_ERR_INVALID, "null runner");
    CUDA_TRY(cudaSetDevice(r->device));
    if(!agreed || r->nearPeerDone.size() != r->world) {
        r->dropNear();
        r->lagStale = true;
        return B200_OK;
    }
    for(uint32_t p = 0; p < r->world; p++) {
        if(!r->nearPeerDone[p]) return fail(B200_ERR_STATE, "the rows held by process %u have not been imported", p);
        if(p != r->rank && !r->peerArena[p]) return fail(B200_ERR_STATE, "exchange arena of rank %u has not been opened", p);
    }
    if(r->nearTable) cudaFree(r->nearTable);
    r->nearTable = nullptr;
    // the rings of every process as this process sees them: same offset in the peer's arena
    std::vector<NearRing> rings((size_t)r->world * r->numRings);
    for(uint32_t p = 0; p < r->world; p++) {
        for(uint32_t i = 0; i < r->numRings; i++) {
            NearRing ring = r->nearRingsHost[i];
            if(p != r->rank) {
                ring.den_delay = reinterpret_cast<float*>(r->peerArena[p] + (reinterpret_cast<unsigned char*>(ring.den_delay) - r->arena));
            }
            rings[(size_t)p * r->numRings + i] = ring;
        }
    }
    if(r->nearRings) cudaFree(r->nearRings);
    if(r->nearSpaces) cudaFree(r->nearSpaces);
    CUDA_TRY(cudaMalloc(&r->nearRings, sizeof(NearRing) * rings.size()));
    CUDA_TRY(cudaMemcpy(r->nearRings, rings.data(), sizeof(NearRing) * rings.size(), cudaMemcpyHostToDevice));
    CUDA_TRY(cudaMalloc(&r->nearSpaces, sizeof(NearSpace) * r->nearSpacesAll.size()));
    CUDA_TRY(cudaMemcpy(r->nearSpaces, r->nearSpacesAll.data(), sizeof(NearSpace) * r->nearSpacesAll.size(), cudaMemcpyHostToDevice));
    r->emitAgreed = true;
    r->queuesAgreed = r->fusedGrid <= NEAR_QUEUE_COUNT;
    for(uint32_t p = 0; p < r->world; p++) {
        if(r->peerGrid[p] != r->fusedGrid) r->queuesAgreed = false;
    }
    r->lagStale = true;
    return B200_OK;
}

int b200_exchange_configure(b200_runner *r, uint32_t rank, uint32_t world)
{
    if(!r || world == 0 || world > B200_MAX_RANKS || rank >= world) return fail(B200_ERR_INVALID, "bad rank/world");
    if(world > 1 && !r->arena) return fail(B200_ERR_STATE, "no exchange arena");
    r->rank = rank;
    r->world = world;
    r->dirty = true;
    return B200_OK;
}

int b200_array_free(b200_runner *r, void *device_ptr)
{
    auto it = r->arrays.find(device_ptr);
    if(it == r->arrays.end()) return fail(B200_ERR_INVALID, "pointer was not allocated by this runner");
    CUDA_TRY(cudaStreamSynchronize(r->stream));
    CUDA_TRY(cudaFree(device_ptr));
    r->arrays.erase(it);
    return B200_OK;
}

int b200_array_push(b200_runner *r, void *device_ptr, const void *host, size_t bytes)
{
    CUDA_TRY(cudaMemcpyAsync(device_ptr, host, bytes, cudaMemcpyHostToDevice, r->stream));
    CUDA_TRY(cudaStreamSynchronize(r->stream));
    if(touchesDelays(r, device_ptr, bytes)) { r->lagStale = true; r->nearDataStale = true; }
    if(touchesSparse(r, device_ptr, bytes)) r->tiledStale = true;
    return B200_OK;
}

int b200_array_pull(b200_runner *r, void *host, const void *device_ptr, size_t bytes)
{
    CUDA_TRY(cudaMemcpyAsync(host, device_ptr, bytes, cudaMemcpyDeviceToHost, r->stream));
    CUDA_TRY(cudaStreamSynchronize(r->stream));
    return B200_OK;
}

int b200_array_memset(b200_runner *r, void *device_ptr, int value, size_t bytes)
{
    CUDA_TRY(cudaMemsetAsync(device_ptr, value, bytes, r->stream));
    if(touchesDelays(r, device_ptr, bytes)) { r->lagStale = true; r->nearDataStale = true; }
    if(touchesSparse(r, device_ptr, bytes)) r->tiledStale = true;
    return B200_OK;
}

int b200_push_neuron_update_group(b200_runner *r, uint32_t idx, const b200_neuron_group *g)
{
    if(!r || !g) return fail(B200_ERR_INVALID, "null argument");
    if(g->num_psm > B200_MAX_PSM || g->num_cs > B200_MAX_CS) return fail(B200_ERR_INVALID, "too many children");
    if(g->num_delay_slots < 2) return fail(B200_ERR_INVALID, "num_delay_slots must be at least 2");
    if(g->first_neuron + g->num_update > g->num_neurons) return fail(B200_ERR_INVALID, "update slice out of range");
    if(g->first_neuron & 31u) return fail(B200_ERR_INVALID, "first_neuron must be a multiple of 32");
    if(!g->spk_cnt || !g->spk) return fail(B200_ERR_INVALID, "spike arrays missing");
    if(idx >= r->neuronGroups.size()) r->neuronGroups.resize(idx + 1);
    r->neuronGroups[idx] = *g;
    r->dirty = true;
    return B200_OK;
}

int b200_validate_synapse_group(const b200_synapse_group *g)
{
    if(!g) return fail(B200_ERR_INVALID, "null argument");
    if(g->connectivity == B200_CONN_SPARSE) {
        if(!g->row_length || !g->ind) return fail(B200_ERR_INVALID, "SPARSE group without row_length/ind");
        if(g->ind_bytes != 1 && g->ind_bytes != 2 && g->ind_bytes != 4) return fail(B200_ERR_INVALID, "bad ind_bytes");
    }
    if(g->connectivity == B200_CONN_BITMASK) {
        if(!g->gp || (g->row_stride & 31u)) return fail(B200_ERR_INVALID, "BITMASK needs gp and a row stride padded to 32");
        if(g->wu_model != B200_WU_STATIC_PULSE_CONSTANT_WEIGHT) return fail(B200_ERR_INVALID, "BITMASK carries no per-synapse variables");
    }
    if(g->connectivity == B200_CONN_PROCEDURAL) {
        if(g->proc_connect != B200_CONNECT_FIXED_PROBABILITY && g->proc_connect != B200_CONNECT_FIXED_PROBABILITY_NO_AUTAPSE &&
           g->proc_connect != B200_CONNECT_FIXED_NUMBER_POST_WITH_REPLACEMENT) {
            return fail(B200_ERR_INVALID, "PROCEDURAL connectivity needs a snippet that builds rows without stored lengths");
        }
        if(g->wu_model != B200_WU_STATIC_PULSE && g->wu_model != B200_WU_STATIC_PULSE_CONSTANT_WEIGHT) {
            return fail(B200_ERR_INVALID, "PROCEDURAL connectivity supports StaticPulse and StaticPulseConstantWeight");
        }
        if(!g->row_stride) return fail(B200_ERR_INVALID, "PROCEDURAL group without a row stride (longest row)");
    }
    if(g->wu_model != B200_WU_STATIC_PULSE_CONSTANT_WEIGHT && g->connectivity != B200_CONN_PROCEDURAL && !g->g) {
        return fail(B200_ERR_INVALID, "weight array missing");
    }
    if(g->wu_model == B200_WU_STATIC_PULSE_DENDRITIC_DELAY && (!g->d || !g->den_delay || !g->max_den_delay)) {
        return fail(B200_ERR_INVALID, "dendritic delay group without d/den_delay");
    }
    // the kernels switch on max_den_delay: a ring depth means "read d, add into den_delay"
    if(g->max_den_delay && (!g->den_delay || (!g->d && g->connectivity != B200_CONN_PROCEDURAL))) {
        return fail(B200_ERR_INVALID, "max_den_delay set but d or den_delay missing");
    }
    if(g->max_den_delay && g->wu_model != B200_WU_STATIC_PULSE_DENDRITIC_DELAY && g->connectivity != B200_CONN_PROCEDURAL) {
        return fail(B200_ERR_INVALID, "max_den_delay set on a weight update model that does not call addToPostDelay");
    }
    if((g->max_den_delay || g->wu_model == B200_WU_STATIC_PULSE_DENDRITIC_DELAY) &&
       (g->connectivity == B200_CONN_BITMASK || g->connectivity == B200_CONN_DENSE)) {
        return fail(B200_ERR_INVALID, "dendritic delay is supported on SPARSE connectivity only");
    }
    if(!g->max_den_delay && !g->out_post) return fail(B200_ERR_INVALID, "out_post missing");
    if(g->connectivity == B200_CONN_SPARSE) {
        // rows are read as aligned groups of four synapses counted from the array base
        if(g->g && ((uintptr_t)g->g & 15u)) return fail(B200_ERR_INVALID, "g must be 16-byte aligned");
        if((uintptr_t)g->ind & (4u * g->ind_bytes - 1u)) return fail(B200_ERR_INVALID, "ind must be aligned to four indices");
        if(g->d && ((uintptr_t)g->d & 3u)) return fail(B200_ERR_INVALID, "d must be 4-byte aligned");
    }
    if(g->wu_model == B200_WU_STDP) {
        if(!g->src_spike_times || !g->trg_spike_times || !g->trg_spk || !g->trg_spk_cnt) {
            return fail(B200_ERR_INVALID, "learning group without spike times");
        }
        if(g->connectivity == B200_CONN_SPARSE && (!g->col_length || !g->remap)) {
            return fail(B200_ERR_INVALID, "learning SPARSE group without remap");
        }
        if(g->back_prop_delay + 2 > g->trg_delay_slots) {
            return fail(B200_ERR_INVALID, "back-propagation delay exceeds the target spike queue");
        }
    }
    if(g->axonal_delay + 2 > g->src_delay_slots) return fail(B200_ERR_INVALID, "axonal delay exceeds the source spike queue");
    return B200_OK;
}

int b200_push_synapse_group(b200_runner *r, uint32_t idx, const b200_synapse_group *g)
{
    if(!r || !g) return fail(B200_ERR_INVALID, "null argument");
    if(const int e = b200_validate_synapse_group(g)) return e;
    if(idx >= r->synapseGroups.size()) r->synapseGroups.resize(idx + 1);
    r->synapseGroups[idx] = *g;
    r->dirty = true;
    return B200_OK;
}

int b200_push_custom_update(b200_runner *r, const char *name, uint32_t idx, const b200_custom_update_group *u)
{
    if(!r || !name || !u) return fail(B200_ERR_INVALID, "null argument");
    auto &v = r->customUpdates[name];
    if(idx >= v.size()) v.resize(idx + 1);
    v[idx] = *u;
    return B200_OK;
}

int b200_set_option(b200_runner *r, const char *name, double value)
{
    const std::string n(name);
    if(n == "spike_lanes") r->spikeLanes = std::max(1u, (unsigned int)value);
    else if(n == "count_events") r->countEvents = (value != 0.0);
    else if(n == "use_graph") r->useGraph = (value != 0.0);
    else if(n == "use_fused") r->useFused = (value != 0.0);
    else if(n == "use_lag") { r->useLag = (value != 0.0); r->lagStale = true; }
    else if(n == "use_split") { r->useSplit = (value != 0.0); r->lagStale = true; }
    else if(n == "use_near_queues") r->useNearQueues = (value != 0.0);
    else if(n == "near_queue_words") {
        if(value < 2.0 || value > (double)NEAR_QUEUE_WORDS) return fail(B200_ERR_INVALID, "near_queue_words must lie in [2, %u]", NEAR_QUEUE_WORDS);
        r->queueWords = (unsigned int)value;
    }
    else if(n == "use_emit") { r->useEmit = (value != 0.0); r->lagStale = true; }
    else if(n == "stream_warps") { r->streamWarpsWanted = (int)value; r->lagStale = true; }
    else if(n == "lag_agreed") { r->lagAgreed = (value != 0.0); r->lagStale = true; }
    else if(n == "rescan_delays") r->lagStale = true;
    else if(n == "fused_profile") {
        // (the per-CTA cycle counters are allocated here, not on the time-step path)
        r->fusedProfile = (value != 0.0);
        if(r->fusedProfile && !r->fusedCtaCycles) {
            CUDA_TRY(cudaSetDevice(r->device));
            CUDA_TRY(cudaMalloc(&r->fusedCtaCycles, sizeof(unsigned long long) * 5 * PROFILE_MAX_CTAS));
            CUDA_TRY(cudaMemset(r->fusedCtaCycles, 0, sizeof(unsigned long long) * 5 * PROFILE_MAX_CTAS));
        }
    }
    else if(n == "fused_blocks_per_sm") { r->fusedBlocksPerSM = (unsigned int)value; r->dirty = true; }
    else if(n == "graph_steps") r->graphSteps = std::max(1u, (unsigned int)value);
    else if(n == "barrier_spin_limit" || n == "exchange_spin_limit" || n == "stream_wait_cycles") {
        // limits of the waits inside the persistent kernels (polls, polls, SM cycles); a wait that runs out
        // makes the launch return early and b200_synchronize report it
        if(value < 1.0) return fail(B200_ERR_INVALID, "%s must be at least 1", name);
        const unsigned long long v = (unsigned long long)value;
        unsigned long long *dst = (n == "barrier_spin_limit") ? &r->state->barrier_spin_limit
                                : (n == "exchange_spin_limit") ? &r->state->exchange_spin_limit
                                : reinterpret_cast<unsigned long long*>(&r->state->stream_wait_cycles);
        CUDA_TRY(cudaStreamSynchronize(r->stream));
        CUDA_TRY(cudaMemcpy(dst, &v, sizeof(v), cudaMemcpyHostToDevice));
    }
    else if(n == "use_tiled") { r->useTiled = (value != 0.0); r->tiledStale = true; }
    else if(n == "tiled_min_events") r->tiledMinEvents = (float)value;
    else if(n == "tiled_ticket_events") { r->tiledTicketEvents = std::max(1.0f, (float)value); r->dropGraph(); }
    else if(n == "tiled_ticket_cost") { r->tiledTicketCost = std::max(0.0f, (float)value); r->dropGraph(); }
    else return fail(B200_ERR_INVALID, "unknown option %s", name);
    r->dropGraph();
    return B200_OK;
}

int b200_initialize(b200_runner *r)
{
    CUDA_TRY(cudaSetDevice(r->device));
    return prepare(r);
}

int b200_initialize_sparse(b200_runner *r)
{
    CUDA_TRY(cudaSetDevice(r->device));
    return prepare(r);
}

int b200_init_var(b200_runner *r, void *device_ptr, uint32_t elem_bytes, uint64_t count,
                  uint32_t snippet, const float *params, uint32_t rng_stream)
{
    r->lagStale = true;
    r->tiledStale = true;
    InitParams prm{};
    for(int i = 0; i < 4; i++) prm.p[i] = params ? params[i] : 0.0f;
    const unsigned int blocks = (unsigned int)std::min<uint64_t>((count + INIT_BLOCK - 1) / INIT_BLOCK, 148u * 32u);
    if(count == 0) return B200_OK;
    if(elem_bytes == 4) {
        initVarKernel<float><<<blocks, INIT_BLOCK, 0, r->stream>>>((float*)device_ptr, count, snippet, prm, r->seed, rng_stream);
    }
    else if(elem_bytes == 1) {
        initVarKernel<uint8_t><<<blocks, INIT_BLOCK, 0, r->stream>>>((uint8_t*)device_ptr, count, snippet, prm, r->seed, rng_stream);
    }
    else return fail(B200_ERR_INVALID, "element size %u not supported", elem_bytes);
    r->launches++;
    CUDA_TRY(cudaPeekAtLastError());
    return B200_OK;
}

int b200_init_sparse_connectivity(b200_runner *r, uint32_t snippet, const float *params,
                                  uint32_t num_src, uint32_t num_trg, uint32_t row_stride,
                                  uint32_t ind_bytes, uint32_t trg_begin, uint32_t trg_end,
                                  uint32_t *row_length, void *ind, uint32_t rng_stream)
{
    r->lagStale = true;
    r->tiledStale = true;
    if(trg_end > num_trg || trg_begin >= trg_end) return fail(B200_ERR_INVALID, "bad target range");
    InitParams prm{};
    for(int i = 0; i < 4; i++) prm.p[i] = params ? params[i] : 0.0f;
    return withIndType(ind_bytes, [&](auto tag) -> int {
        using IndT = decltype(tag);
        if(snippet == B200_CONNECT_FIXED_NUMBER_PRE_WITH_REPLACEMENT) {
            CUDA_TRY(cudaMemsetAsync(row_length, 0, sizeof(uint32_t) * num_src, r->stream));
            const unsigned int n = trg_end - trg_begin;
            initFixedNumberPreKernel<IndT><<<(n + INIT_BLOCK - 1) / INIT_BLOCK, INIT_BLOCK, 0, r->stream>>>(
                (unsigned int)prm.p[0], num_src, row_stride, trg_begin, trg_end, row_length, ind, r->seed, rng_stream, r->state);
        }
        else {
            initSparseConnectivityKernel<IndT><<<(num_src + INIT_BLOCK - 1) / INIT_BLOCK, INIT_BLOCK, 0, r->stream>>>(
                snippet, prm, num_src, row_stride, trg_begin, trg_end, row_length, ind, r->seed, rng_stream, r->state);
        }
        r->launches++;
        CUDA_TRY(cudaPeekAtLastError());
        return B200_OK;
    });
}

int b200_init_sparse_vars(b200_runner *r, const uint32_t *row_length, uint32_t num_src,
                          uint32_t row_stride, void *device_ptr, uint32_t elem_bytes,
                          uint32_t snippet, const float *params, uint32_t rng_stream)
{
    r->lagStale = true;
    r->tiledStale = true;
    InitParams prm{};
    for(int i = 0; i < 4; i++) prm.p[i] = params ? params[i] : 0.0f;
    const uint64_t total = (uint64_t)num_src * row_stride;
    if(total == 0) return B200_OK;
    const unsigned int blocks = (unsigned int)std::min<uint64_t>((total + INIT_BLOCK - 1) / INIT_BLOCK, 148u * 32u);
    if(elem_bytes == 4) {
        initSparseVarKernel<float><<<blocks, INIT_BLOCK, 0, r->stream>>>((float*)device_ptr, row_length, num_src, row_stride, snippet, prm, r->seed, rng_stream);
    }
    else if(elem_bytes == 1) {
        initSparseVarKernel<uint8_t><<<blocks, INIT_BLOCK, 0, r->stream>>>((uint8_t*)device_ptr, row_length, num_src, row_stride, snippet, prm, r->seed, rng_stream);
    }
    else return fail(B200_ERR_INVALID, "element size %u not supported", elem_bytes);
    r->launches++;
    CUDA_TRY(cudaPeekAtLastError());
    return B200_OK;
}

int b200_build_remap(b200_runner *r, const uint32_t *row_length, const void *ind, uint32_t ind_bytes,
                     uint32_t num_src, uint32_t num_trg, uint32_t row_stride, uint32_t col_stride,
                     uint32_t *col_length, uint32_t *remap)
{
    const uint64_t total = (uint64_t)num_src * row_stride;
    CUDA_TRY(cudaMemsetAsync(col_length, 0, sizeof(uint32_t) * num_trg, r->stream));
    if(total == 0) return B200_OK;
    const unsigned int blocks = (unsigned int)std::min<uint64_t>((total + INIT_BLOCK - 1) / INIT_BLOCK, 148u * 32u);
    return withIndType(ind_bytes, [&](auto tag) -> int {
        using IndT = decltype(tag);
        buildRemapKernel<IndT><<<blocks, INIT_BLOCK, 0, r->stream>>>(row_length, ind, num_src, num_trg, row_stride,
                                                                     col_stride, col_length, remap, r->state);
        r->launches++;
        CUDA_TRY(cudaPeekAtLastError());
        return B200_OK;
    });
}

int b200_update_synapses(b200_runner *r)
{
    int e = prepare(r);
    if(e) return e;
    e = ensureTiled(r);
    if(e) return e;
    return enqueueSynapses(r, false, true);
}

int b200_update_neurons(b200_runner *r, uint64_t num_recording_timesteps)
{
    int e = prepare(r);
    if(e) return e;
    e = enqueueNeurons(r, num_recording_timesteps, false);
    if(e == B200_OK) {
        r->hostTimestep++;
        r->hostStepsDone++;
    }
    return e;
}

int b200_step_time(b200_runner *r, uint64_t num_steps, uint64_t num_recording_timesteps)
{
    int e = prepare(r);
    if(e) return e;
    uint64_t left = num_steps;
    if(r->sharded() && !(r->useFused && r->fusedEligible && !r->timing)) {
        return fail(B200_ERR_STATE, "a sharded model runs on the persistent kernel only (batch 1, SPARSE "
                                    "non-learning groups, per-kernel timing off)");
    }
    if(r->useFused && r->fusedEligible && !r->timing) {
        while(left) {
            const uint64_t n = std::min<uint64_t>(left, 1ull << 20);
            e = launchFused(r, n, num_recording_timesteps);
            if(e) return e;
            left -= n;
        }
    }
    else if((e = ensureTiled(r)) != B200_OK || (e = pollPeak(r)) != B200_OK) {
        return e;
    }
    else if(r->useGraph && !r->timing && num_steps >= 2) {
        const unsigned int len = (unsigned int)std::min<uint64_t>(num_steps, r->graphSteps);
        if(!r->graphExec || r->graphLen > num_steps || r->graphNumRec != num_recording_timesteps ||
           (r->graphLen != len && r->graphLen != r->graphSteps)) {
            e = buildGraph(r, len, num_recording_timesteps);
            if(e) return e;
        }
        while(left >= r->graphLen) {
            CUDA_TRY(cudaGraphLaunch(r->graphExec, r->stream));
            r->launches += (unsigned long long)r->graphLen * kernelsPerStep(r);
            left -= r->graphLen;
        }
    }
    for(; left; left--) {
        e = enqueueStep(r, num_recording_timesteps, false);
        if(e) return e;
    }
    if(r->tiledReady && !(r->useFused && r->fusedEligible && !r->timing)) {
        e = fetchPeak(r);
        if(e) return e;
    }
    r->hostTimestep += num_steps;
    r->hostStepsDone += num_steps;
    return B200_OK;
}


int b200_nccl_unique_id(void *id_128_bytes)
{
    if(!id_128_bytes) return fail(B200_ERR_INVALID, "null id buffer");
    NcclApi *api = ncclApi();
    if(!api) return fail(B200_ERR_STATE, "libnccl.so.2 could not be loaded: %s", dlerror());
    NcclId id;
    NCCL_TRY(api, api->getUniqueId(&id));
    memcpy(id_128_bytes, &id, sizeof(id));
    return B200_OK;
}

int b200_nccl_init(b200_runner *r, const void *id_128_bytes, uint32_t rank, uint32_t world)
{
    if(!r || !id_128_bytes || world == 0 || rank >= world) return fail(B200_ERR_INVALID, "bad arguments to b200_nccl_init");
    if(r->ncclComm) return fail(B200_ERR_STATE, "the communicator has already been created");
    NcclApi *api = ncclApi();
    if(!api) return fail(B200_ERR_STATE, "libnccl.so.2 could not be loaded: %s", dlerror());
    CUDA_TRY(cudaSetDevice(r->device));
    NcclId id;
    memcpy(&id, id_128_bytes, sizeof(id));
    NCCL_TRY(api, api->commInitRank(&r->ncclComm, (int)world, id, (int)rank));
    r->ncclWorld = world;
    return B200_OK;
}

// A custom update group.  `phases`: bit 0 reduce over the batch, bit 1 write back.  With a communicator
// (data-parallel run: every process holds a share of the batch) the reduced values of ALL updates of the
// group are packed into one buffer, sums first, combined with one all-reduce per operation on the
// runner's stream, and written back from there: no host synchronisation anywhere.
static int runCustomUpdate(b200_runner *r, const char *name, unsigned int phases)
{
    auto it = r->customUpdates.find(name);
    if(it == r->customUpdates.end()) return fail(B200_ERR_INVALID, "no custom update group '%s'", name);
    ScopedTimer tm(r, std::string("custom_update_") + name, false);
    const bool combine = r->ncclComm && r->ncclWorld > 1 && phases == 3u;
    auto blocksFor = [](uint64_t n) { return (unsigned int)std::min<uint64_t>((n + REDUCE_BLOCK - 1) / REDUCE_BLOCK, 148u * 16u); };
    if(!combine) {
        for(const auto &u : it->second) {
            if(u.num_elements == 0) continue;
            batchReduceKernel<<<blocksFor(u.num_elements), REDUCE_BLOCK, 0, r->stream>>>(u, r->batch, phases, nullptr);
            r->launches++;
        }
        CUDA_TRY(cudaPeekAtLastError());
        return B200_OK;
    }
    // layout of the packed buffer: every update's segment starts on a 16-byte boundary
    std::vector<size_t> offset(it->second.size(), 0);
    size_t total = 0, sums = 0;
    for(int pass = 0; pass < 2; pass++) {
        for(size_t i = 0; i < it->second.size(); i++) {
            const auto &u = it->second[i];
            if((u.op == B200_REDUCE_SUM) != (pass == 0)) continue;
            offset[i] = total;
            total += (u.num_elements + 3) & ~(uint64_t)3;
        }
        if(pass == 0) sums = total;
    }
    if(total > r->reducePackedElements) {
        CUDA_TRY(cudaStreamSynchronize(r->stream));
        if(r->reducePacked) CUDA_TRY(cudaFree(r->reducePacked));
        r->reducePacked = nullptr;
        CUDA_TRY(cudaMalloc(&r->reducePacked, sizeof(float) * total));
        CUDA_TRY(cudaMemsetAsync(r->reducePacked, 0, sizeof(float) * total, r->stream));
        r->reducePackedElements = total;
    }
    for(size_t i = 0; i < it->second.size(); i++) {
        const auto &u = it->second[i];
        if(u.num_elements == 0) continue;
        batchReduceKernel<<<blocksFor(u.num_elements), REDUCE_BLOCK, 0, r->stream>>>(u, r->batch, 1u, r->reducePacked + offset[i]);
        r->launches++;
    }
    CUDA_TRY(cudaPeekAtLastError());
    NcclApi *api = ncclApi();
    if(sums) NCCL_TRY(api, api->allReduce(r->reducePacked, r->reducePacked, sums, NCCL_FLOAT32, NCCL_SUM, r->ncclComm, r->stream));
    if(total > sums) NCCL_TRY(api, api->allReduce(r->reducePacked + sums, r->reducePacked + sums, total - sums, NCCL_FLOAT32, NCCL_MAX, r->ncclComm, r->stream));
    for(size_t i = 0; i < it->second.size(); i++) {
        const auto &u = it->second[i];
        if(u.num_elements == 0) continue;
        batchReduceKernel<<<blocksFor(u.num_elements), REDUCE_BLOCK, 0, r->stream>>>(u, r->batch, 2u, r->reducePacked + offset[i]);
        r->launches++;
    }
    CUDA_TRY(cudaPeekAtLastError());
    return B200_OK;
}

int b200_custom_update(b200_runner *r, const char *name)
{
    return runCustomUpdate(r, name, 3u);
}

int b200_custom_update_reduce(b200_runner *r, const char *name)
{
    return runCustomUpdate(r, name, 1u);
}

int b200_custom_update_broadcast(b200_runner *r, const char *name)
{
    return runCustomUpdate(r, name, 2u);
}

int b200_synchronize(b200_runner *r)
{
    CUDA_TRY(cudaStreamSynchronize(r->stream));
    StepState s;
    CUDA_TRY(cudaMemcpy(&s, r->state, sizeof(s), cudaMemcpyDeviceToHost));
    if(s.error) {
        const unsigned int err = s.error;
        cudaMemset(&r->state->error, 0, sizeof(unsigned int));
        return fail(B200_ERR_DEVICE_CHECK, "device-side check failed (flags 0x%x:%s%s%s%s%s)", err,
                    (err & ERR_SPIKE_OVERFLOW) ? " spike list overflow" : "",
                    (err & ERR_IND_RANGE) ? " index or row length out of range" : "",
                    (err & ERR_DELAY_RANGE) ? " a synapse arriving in the same step appeared after the schedule was chosen (option rescan_delays)" : "",
                    (err & ERR_BARRIER_TIMEOUT) ? " grid barrier timed out" : "",
                    (err & ERR_EXCHANGE_TIMEOUT) ? " spikes of another process did not arrive in time" : "");
    }
    return B200_OK;
}

int b200_get_timestep(b200_runner *r, uint64_t *timestep)
{
    *timestep = r->hostTimestep;
    return B200_OK;
}

int b200_set_timestep(b200_runner *r, uint64_t timestep)
{
    CUDA_TRY(cudaStreamSynchronize(r->stream));
    const unsigned long long t = timestep;
    CUDA_TRY(cudaMemcpy(&r->state->timestep, &t, sizeof(t), cudaMemcpyHostToDevice));
    r->hostTimestep = timestep;
    return B200_OK;
}

int b200_get_steps_done(b200_runner *r, uint64_t *steps)
{
    *steps = r->hostStepsDone;
    return B200_OK;
}

int b200_get_counter(b200_runner *r, const char *name, uint64_t *value)
{
    const std::string n(name);
    if(n == "stream_warps") {
        int e = prepare(r);
        if(e) return e;
        if(r->fusedEligible && r->lagStale) {
            e = refreshSchedule(r);
            if(e) return e;
        }
        *value = r->streamWarps;
        return B200_OK;
    }
    if(n == "schedule") {
        // of the next persistent launch: 0 everything before the neuron update, 1 only the synapses that
        // arrive in the same step before it (split delivery), 2 spikes one step late (one barrier per step)
        int e = prepare(r);
        if(e) return e;
        if(r->fusedEligible && r->lagStale) {
            e = refreshSchedule(r);
            if(e) return e;
        }
        *value = (uint64_t)r->schedule;
        return B200_OK;
    }
    if(n == "tiled_armed") {
        // whether the next block of steps on the one-launch-per-kernel path launches the tiled kernels
        *value = tiledActive(r) ? 1u : 0u;
        return B200_OK;
    }
    if(n == "tiled_ready" || n == "tiled_synapses" || n == "heavy") {
        // the target-tiled copy of the SPARSE groups (built when the one-launch-per-kernel path is first
        // used) / the verdict of the last step's event estimate
        if(n == "heavy") {
            unsigned int h = 0;
            CUDA_TRY(cudaStreamSynchronize(r->stream));
            CUDA_TRY(cudaMemcpy(&h, &r->state->heavy, sizeof(h), cudaMemcpyDeviceToHost));
            *value = h;
            return B200_OK;
        }
        int e = prepare(r);
        if(!e) e = ensureTiled(r);
        if(e) return e;
        *value = (n == "tiled_ready") ? (r->tiledReady ? 1u : 0u) : r->tiledSynapses;
        return B200_OK;
    }
    if(n == "lag_eligible" || n == "lag") {
        // whether this process may deliver spikes one step late (scans the delay arrays if
        // they changed) / whether its next persistent launch will
        int e = prepare(r);
        if(e) return e;
        if(r->fusedEligible && r->lagStale) {
            e = refreshSchedule(r);
            if(e) return e;
        }
        const bool can = r->useLag && r->fusedEligible && r->lagEligible;
        *value = (n == "lag") ? (r->useFused && r->fusedEligible && r->schedule == b200_runner::LAG) : can;
        return B200_OK;
    }
    CUDA_TRY(cudaStreamSynchronize(r->stream));
    StepState s;
    CUDA_TRY(cudaMemcpy(&s, r->state, sizeof(s), cudaMemcpyDeviceToHost));
    if(n == "synaptic_events") *value = s.synaptic_events;
    else if(n == "spikes") *value = s.spikes;
    else if(n == "cycles_presynaptic") *value = s.phase_cycles[0];
    else if(n == "cycles_barrier_a") *value = s.phase_cycles[1];
    else if(n == "cycles_neuron") *value = s.phase_cycles[2];
    else if(n == "cycles_barrier_b") *value = s.phase_cycles[3];
    else if(n.size() >= 6 && n.size() <= 7 && n.compare(0, 5, "probe") == 0 && atoi(n.c_str() + 5) >= 0 && atoi(n.c_str() + 5) < 12 &&
            isdigit((unsigned char)n[5])) *value = s.probe[atoi(n.c_str() + 5)];
    else if(n == "timestep") *value = s.timestep;
    else if(n == "steps_done") *value = s.steps_done;
    else return fail(B200_ERR_INVALID, "unknown counter %s", name);
    return B200_OK;
}

/* Per-CTA phase cycles of the persistent kernel (option "fused_profile"): out[cta*4 + phase]. */
int b200_get_cta_cycles(b200_runner *r, uint64_t *out, uint32_t max_ctas, uint32_t *num_ctas)
{
    *num_ctas = 0;
    if(!r->fusedCtaCycles) return B200_OK;
    CUDA_TRY(cudaStreamSynchronize(r->stream));
    const uint32_t n = std::min<uint32_t>(max_ctas, r->fusedGrid);
    CUDA_TRY(cudaMemcpy(out, r->fusedCtaCycles, sizeof(uint64_t) * 4 * n, cudaMemcpyDeviceToHost));
    if(max_ctas >= 2 * r->fusedGrid) {
        // trailing block: cycles from step start to the spike-header barrier
        CUDA_TRY(cudaMemcpy(out + 4ull * n, r->fusedCtaCycles + 4ull * r->fusedGrid, sizeof(uint64_t) * n, cudaMemcpyDeviceToHost));
    }
    *num_ctas = n;
    return B200_OK;
}

/* Which time-step path b200_step_time will take: 2 target-stationary persistent kernel,
 * 1 persistent kernel with global reductions, 0 one launch per kernel.  `why` (may be NULL)
 * receives the reason the faster paths were not chosen. */
int b200_get_step_path(b200_runner *r, int *path, char *why, size_t why_bytes)
{
    const int e = prepare(r);
    if(e) return e;
    *path = (r->useFused && r->fusedEligible) ? 1 : 0;
    if(why && why_bytes) snprintf(why, why_bytes, "%s", r->fusedEligible ? "" : "batch > 1, or groups that are not SPARSE and non-learning");
    return B200_OK;
}

int b200_enable_timing(b200_runner *r, int enabled)
{
    r->timing = (enabled != 0);
    return B200_OK;
}

int b200_get_timer(b200_runner *r, const char *name, double *seconds)
{
    auto it = r->timers.find(name);
    *seconds = (it == r->timers.end()) ? 0.0 : it->second.seconds;
    return B200_OK;
}

int b200_reset_timers(b200_runner *r)
{
    r->timers.clear();
    return B200_OK;
}

int b200_get_kernel_launches(b200_runner *r, uint64_t *launches)
{
    *launches = r->launches;
    return B200_OK;
}

// Time `num_steps` steps with CUDA events recorded on the runner's own stream
// (events of another stream would not see this work).  Synchronises.
int b200_step_time_timed(b200_runner *r, uint64_t num_steps, uint64_t num_recording_timesteps, float *milliseconds)
{
    int e = prepare(r);
    if(e) return e;
    CUDA_TRY(cudaStreamSynchronize(r->stream));
    CUDA_TRY(cudaEventRecord(r->evC, r->stream));
    e = b200_step_time(r, num_steps, num_recording_timesteps);
    if(e) return e;
    CUDA_TRY(cudaEventRecord(r->evD, r->stream));
    CUDA_TRY(cudaEventSynchronize(r->evD));
    CUDA_TRY(cudaEventElapsedTime(milliseconds, r->evC, r->evD));
    return B200_OK;
}

int b200_compact_words(b200_runner *r, const uint32_t *words, uint64_t num_words, uint32_t base_index,
                       void *pairs, uint32_t capacity, uint32_t *counter)
{
    if(!r || !words || !pairs || !counter) return fail(B200_ERR_INVALID, "null argument to b200_compact_words");
    if(base_index + num_words > 0xFFFFFFFFull) return fail(B200_ERR_INVALID, "word indices beyond 32 bits");
    if(num_words == 0) return B200_OK;
    CUDA_TRY(cudaSetDevice(r->device));
    const unsigned int blocks = (unsigned int)std::min<uint64_t>((num_words + 255) / 256, 148u * 8u);
    compactWordsKernel<<<blocks, 256, 0, r->stream>>>(words, num_words, base_index, static_cast<uint2*>(pairs), capacity, counter);
    CUDA_TRY(cudaPeekAtLastError());
    r->launches++;
    return B200_OK;
}

int b200_timed_begin(b200_runner *r)
{
    if(!r) return fail(B200_ERR_INVALID, "null runner");
    int e = prepare(r);
    if(e) return e;
    CUDA_TRY(cudaStreamSynchronize(r->stream));
    CUDA_TRY(cudaEventRecord(r->evC, r->stream));
    return B200_OK;
}

int b200_timed_end(b200_runner *r, float *milliseconds)
{
    if(!r || !milliseconds) return fail(B200_ERR_INVALID, "null argument");
    CUDA_TRY(cudaEventRecord(r->evD, r->stream));
    CUDA_TRY(cudaEventSynchronize(r->evD));
    CUDA_TRY(cudaEventElapsedTime(milliseconds, r->evC, r->evD));
    return B200_OK;
}

}   // extern "C"
