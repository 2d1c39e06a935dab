/* genn_b200.h - C ABI of the B200-native simulation backend.
 *
 * The reference (GeNN 5.4.0) reaches its per-timestep path through the C
 * symbols of a generated librunner.so which its runtime looks up by name
 * (src/genn/genn/runtime/runtime.cc:81-119): allocateMem, freeMem, initialize,
 * initializeSparse, stepTime, update<CustomUpdateGroup>, one
 * pushMerged<Kind>Group<i>ToDevice per merged group and the *Time counters.
 * Those symbols are specific to one generated model.  This library exports the
 * same surface once, for every model built from the built-in neuron,
 * postsynaptic, current-source and weight-update models: a runner object
 * stands for one loaded librunner.so, a group descriptor stands for one
 * element of a merged-group struct array, and the push functions register it.
 *
 * All pointers inside descriptors are DEVICE pointers obtained from
 * b200_array_alloc (the counterpart of BackendBase::createArray,
 * include/genn/genn/code_generator/backendBase.h:305-312) unless stated
 * otherwise.  All functions return 0 on success and a non-zero b200_status on
 * failure; b200_last_error() then describes the failure.  Nothing here
 * allocates or frees device memory inside the time-step path.
 *
 * Array layouts are the reference's: neuron variables [batch][N]; spike lists
 * spk_cnt[batch][slots], spk[batch][slots][N]; SPARSE connectivity as ragged
 * rows row_length[numPre], ind[numPre*row_stride] with per-synapse variables
 * indexed alike; BITMASK as 32-bit words, bit (pre*row_stride + post) counted
 * from the MSB, row_stride padded to 32; DENSE row-major [numPre][numPost];
 * dendritic delay ring den_delay[batch][D][N].
 */
#ifndef GENN_B200_H
#define GENN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_MAX_PSM     8   /* fused incoming postsynaptic models per neuron group */
#define B200_MAX_CS      4   /* current sources per neuron group */
#define B200_MAX_PARAMS  8
#define B200_MAX_VARS    4
#define B200_MAX_RANKS   8   /* processes (one per GPU) a sharded model may span */

typedef enum b200_status {
    B200_OK = 0,
    B200_ERR_CUDA = 1,          /* a CUDA runtime call failed */
    B200_ERR_INVALID = 2,       /* bad argument or descriptor */
    B200_ERR_STATE = 3,         /* call made in the wrong lifecycle state */
    B200_ERR_DEVICE_CHECK = 4   /* a kernel reported a failed bounds check */
} b200_status;

/* neuronModels.h:163-325 */
typedef enum b200_neuron_model {
    B200_NEURON_LIF = 0,              /* parameter and variable order: see b200_neuron_group */
    B200_NEURON_IZHIKEVICH = 1,
    B200_NEURON_SPIKE_SOURCE_ARRAY = 2,
    B200_NEURON_POISSON = 3
} b200_neuron_model;

/* postsynapticModels.h:93-151 */
typedef enum b200_psm_model {
    B200_PSM_EXP_CURR = 0,            /* params: init, expDecay */
    B200_PSM_EXP_COND = 1,            /* params: expDecay, E */
    B200_PSM_DELTA_CURR = 2
} b200_psm_model;

/* currentSourceModels.h:60-129 */
typedef enum b200_cs_model {
    B200_CS_DC = 0,                   /* params: amp */
    B200_CS_POISSON_EXP = 1           /* params: Init, ExpDecay, ExpMinusLambda, lambda; var0: current */
} b200_cs_model;

/* weightUpdateModels.h:236-368 */
typedef enum b200_wu_model {
    B200_WU_STATIC_PULSE = 0,                 /* addToPost(g) */
    B200_WU_STATIC_PULSE_CONSTANT_WEIGHT = 1, /* params: g */
    B200_WU_STATIC_PULSE_DENDRITIC_DELAY = 2, /* addToPostDelay(g, d) */
    B200_WU_STDP = 3                          /* params: tauPlus, tauMinus, Aplus, Aminus, Wmin, Wmax,
                                                 (axonalDelay+1)*dt, (backPropDelay+1)*dt */
} b200_wu_model;

/* synapseMatrixType.h:9-69 */
typedef enum b200_connectivity {
    B200_CONN_SPARSE = 0,
    B200_CONN_BITMASK = 1,
    B200_CONN_DENSE = 2,
    B200_CONN_PROCEDURAL = 3
} b200_connectivity;

/* initVarSnippet.h:87-261 */
typedef enum b200_var_init {
    B200_INIT_CONSTANT = 0,             /* params: constant */
    B200_INIT_UNIFORM = 1,              /* params: min, max */
    B200_INIT_NORMAL = 2,               /* params: mean, sd */
    B200_INIT_NORMAL_CLIPPED = 3,       /* params: mean, sd, min, max (re-sampled) */
    B200_INIT_NORMAL_CLIPPED_DELAY = 4  /* params: meanTimestep, sdTimestep, minTimestep, maxTimestep; rint */
} b200_var_init;

/* initSparseConnectivitySnippet.h:170-486 */
typedef enum b200_connect_init {
    B200_CONNECT_FIXED_PROBABILITY = 0,                  /* params: prob, 1 / log(1 - prob), sub-rows per row (0 or 1: one;
                                                          * T > 1: targets cut into T ranges, range t drawn from stream
                                                          * element pre * T + t: the reference's threads per spike) */
    B200_CONNECT_FIXED_PROBABILITY_NO_AUTAPSE = 1,
    B200_CONNECT_FIXED_NUMBER_TOTAL_WITH_REPLACEMENT = 2,/* row lengths supplied by the host */
    B200_CONNECT_FIXED_NUMBER_PRE_WITH_REPLACEMENT = 3,  /* params: num (in-degree) */
    B200_CONNECT_FIXED_NUMBER_POST_WITH_REPLACEMENT = 4  /* params: num (out-degree) */
} b200_connect_init;

typedef enum b200_reduce_op { B200_REDUCE_SUM = 0, B200_REDUCE_MAX = 1 } b200_reduce_op;

/* One fused incoming postsynaptic model: the InSynPSM child of a merged
 * neuron-update group (neuronUpdateGroupMerged.cc:66-137). */
typedef struct b200_psm {
    uint32_t model;            /* b200_psm_model */
    uint32_t max_den_delay;    /* ring depth D; 0 = no dendritic delay */
    float    params[4];
    float   *out_post;         /* [batch][N] */
    float   *den_delay;        /* [batch][D][N] or NULL */
} b200_psm;

/* One current source child (neuronUpdateGroupMerged.cc:20-55). */
typedef struct b200_current_source {
    uint32_t model;            /* b200_cs_model */
    uint32_t rng_stream;       /* distinguishes RNG consumers in the Philox counter */
    float    params[4];
    float   *var0;             /* [batch][N] or NULL */
} b200_current_source;

/* One element of the merged neuron-update group array
 * (backendSIMT.cc:405-662, neuronUpdateGroupMerged.cc:552-773).
 *   LIF params:        Vthresh, Vreset, Vrest, Ioffset, Rmembrane, ExpTC, TauRefrac; vars V, RefracTime
 *   Izhikevich params: a, b, c, d;                                                   vars V, U
 *   SpikeSourceArray:  vars startSpike, endSpike (uint32); egp = spikeTimes
 *   Poisson params:    isi;                                                          vars timeStepToSpike */
typedef struct b200_neuron_group {
    uint32_t model;            /* b200_neuron_model */
    uint32_t num_neurons;
    uint32_t num_delay_slots;  /* spike queue depth: at least longest axonal/back-propagation delay + 2;
                                  + 4 lets the persistent kernel deliver spikes one step late (option "use_lag") */
    uint32_t num_psm;
    uint32_t num_cs;
    uint32_t rng_stream;
    uint32_t first_neuron;     /* this process updates neurons [first_neuron, first_neuron+num_update) */
    uint32_t num_update;
    float    params[B200_MAX_PARAMS];
    void    *vars[B200_MAX_VARS];
    const float *egp;          /* SpikeSourceArray spikeTimes */
    uint32_t *spk_cnt;         /* [batch][slots] */
    uint32_t *spk;             /* [batch][slots][N] */
    float    *spike_times;     /* sT [batch][slots][N] or NULL */
    uint32_t *record_spk;      /* [recordingTimesteps][batch][ceil(num_update/32)] or NULL; neuron first_neuron + j
                                  is bit j%32 of word j/32 (the whole population when the process updates all of it) */
    b200_psm psm[B200_MAX_PSM];
    b200_current_source cs[B200_MAX_CS];
    uint32_t spk_slot_stride;  /* elements between two slots of `spk`; 0 = num_neurons.  A process that
                                  updates a slice of the group keeps a list sized for the slice. */
    uint32_t reserved;
    uint64_t *spk_tag;         /* sharded models: [slots] (step << 32 | count) of this process's section; else NULL */
    uint64_t *spk_wire;        /* sharded models: [slots][spk_slot_stride] (step << 32 | neuron id), the copy of the
                                  spike list that travels between processes; else NULL */
} b200_neuron_group;

/* One element of the merged presynaptic-update group array and, when the
 * weight update model learns, of the merged postsynaptic-update group array
 * (presynapticUpdateStrategySIMT.cc:57-745, backendSIMT.cc:766-803). */
typedef struct b200_synapse_group {
    uint32_t connectivity;     /* b200_connectivity */
    uint32_t wu_model;         /* b200_wu_model */
    uint32_t num_src;
    uint32_t num_trg;
    uint32_t row_stride;       /* SPARSE: max row length; BITMASK: num_trg padded to 32; DENSE: num_trg */
    uint32_t ind_bytes;        /* SPARSE index width: 1, 2 or 4 */
    uint32_t axonal_delay;     /* steps */
    uint32_t back_prop_delay;  /* steps */
    uint32_t src_delay_slots;  /* num_delay_slots of the source / target neuron group */
    uint32_t trg_delay_slots;
    uint32_t max_den_delay;    /* ring depth of the target buffer; 0 = addToPost */
    uint32_t col_stride;       /* max column length (learning only) */
    float    wu_params[B200_MAX_PARAMS];
    const uint32_t *row_length;/* SPARSE [numSrc] */
    const void     *ind;       /* SPARSE [numSrc*row_stride] uint8/uint16/uint32 */
    float          *g;         /* per-synapse weight ([batch] duplicated when the model learns) or NULL */
    const uint8_t  *d;         /* per-synapse dendritic delay or NULL */
    const uint32_t *gp;        /* BITMASK words or NULL */
    const uint32_t *col_length;/* [numTrg] (learning only) */
    const uint32_t *remap;     /* [numTrg*col_stride] row-major synapse index (learning only) */
    const uint32_t *src_spk_cnt;
    const uint32_t *src_spk;
    const uint32_t *trg_spk_cnt;
    const uint32_t *trg_spk;
    const float    *src_spike_times;
    const float    *trg_spike_times;
    float          *out_post;  /* target fused buffer [batch][numTrg] */
    float          *den_delay; /* target ring [batch][D][numTrg] or NULL */
    /* PROCEDURAL: connectivity and weights regenerated per spike */
    uint32_t proc_connect;     /* b200_connect_init */
    uint32_t proc_weight_init; /* b200_var_init */
    uint32_t rng_stream;       /* Philox stream of the connectivity (row r: element r of the stream) */
    uint32_t proc_weight_stream; /* Philox stream of the weights (synapse pre*row_stride + position) */
    float    proc_connect_params[4];
    float    proc_weight_params[4];
    /* Sharded source population: the spike lists of `src_sections` processes lie one after another,
     * section s at src_spk_cnt + s*src_cnt_section_stride and src_spk + s*src_spk_section_stride
     * (elements); ids are indices into the whole population.  0 or 1: a single list. */
    uint32_t src_sections;
    uint32_t src_spk_slot_stride;      /* elements between two slots of one list; 0 = num_src */
    uint64_t src_cnt_section_stride;
    uint64_t src_spk_section_stride;
    const uint64_t *src_spk_tag;       /* sharded: tagged counts, laid out like src_spk_cnt; else NULL */
    const uint64_t *src_spk_wire;      /* sharded: tagged ids, laid out like src_spk; else NULL */
} b200_synapse_group;

/* Batch-reduce custom update (backendSIMT.cc:888-927, 1109-1147):
 * target[e] = op over b of source[b][e]; optionally broadcast back. */
typedef struct b200_custom_update_group {
    uint32_t op;               /* b200_reduce_op */
    uint32_t broadcast;        /* 1: write target[e]*scale back into every source[b][e] */
    uint64_t num_elements;
    float    scale;            /* applied to the reduced value (e.g. 1/batch for a mean) */
    uint32_t reserved;
    float   *source;           /* [batch][E] */
    float   *target;           /* [E] */
} b200_custom_update_group;

typedef struct b200_runner b200_runner;

/* ---- lifecycle: allocateMem / freeMem (generateRunner.cc:223-268) -------- */
int  b200_runner_create(int device, double dt, uint64_t seed, uint32_t batch_size, b200_runner **out);
int  b200_runner_destroy(b200_runner *r);
const char *b200_last_error(void);
int  b200_device_count(int *count);

/* ---- arrays: BackendBase::createArray and Runtime::ArrayBase
 *      (backendBase.h:305-312, runtime.h:95-182) ---------------------------- */
int  b200_array_alloc(b200_runner *r, size_t bytes, void **device_ptr);
int  b200_array_free(b200_runner *r, void *device_ptr);
/* Page-locked host memory for the host side of an array (the reference's Array::allocate
 * uses cudaHostAlloc, src/genn/backends/cuda/backend.cc:88-101). */
int  b200_host_alloc(b200_runner *r, size_t bytes, void **host_ptr);
int  b200_host_free(b200_runner *r, void *host_ptr);
int  b200_array_push(b200_runner *r, void *device_ptr, const void *host, size_t bytes);
int  b200_array_pull(b200_runner *r, void *host, const void *device_ptr, size_t bytes);
int  b200_array_memset(b200_runner *r, void *device_ptr, int value, size_t bytes);
/* Spike recordings are one bit per neuron and time step and almost all zeros (Runtime::pullRecordingBuffersFromDevice,
 * runtime.cc:720-746, copies them whole).  This appends the non-zero 32-bit words of `words` to `pairs` as
 * (base_index + word index, word), 8 bytes each, on the runner's stream; `counter` (a device word the caller has
 * zeroed) counts every non-zero word, also those that found no room below `capacity`: the caller then copies
 * the array itself.  Order of the pairs is arbitrary. */
int  b200_compact_words(b200_runner *r, const uint32_t *words, uint64_t num_words, uint32_t base_index,
                        void *pairs, uint32_t capacity, uint32_t *counter);

/* ---- spike exchange between processes (no counterpart in the reference, which has no model
 *      sharding: backendCUDAHIP.cc uses NCCL for the all-reduce of custom-update results only).
 * A model sharded by postsynaptic neuron over several GPUs of one node exchanges each step's spike
 * lists.  Every process allocates ONE exchange arena, places its spike arrays (all sections) and the
 * tagged counts in it at identical offsets, shares the arena's IPC handle with its peers and opens
 * theirs.  The persistent kernel then writes each spike straight into every peer's arena with peer
 * stores as it is emitted and, once the step's list is final, one count word per population.  Every
 * word on the wire is 64 bits, (step << 32 | payload): a reader polls its OWN memory until the word
 * carries the step it expects, so no ordering between the stores (and no system-scope fence, 1.5 us
 * on this hardware) is needed. -------------------------------------------------------------------- */
int  b200_exchange_alloc(b200_runner *r, size_t bytes, void **device_ptr);
/* The arena is larger than the `bytes` asked for: behind them lie the queues through which the "deliver at
 * emission" schedule sends near synapses between processes.  `bytes` returns the whole size, which a peer
 * registered with b200_exchange_set_peer must provide as well. */
int  b200_exchange_bytes(b200_runner *r, size_t *bytes);
int  b200_exchange_get_handle(b200_runner *r, void *handle_64_bytes);
int  b200_exchange_open_peer(b200_runner *r, uint32_t peer_rank, const void *handle_64_bytes);
/* A peer whose arena is already addressable in THIS process (another runner of the same process, on this
 * device or on one with peer access enabled): registered by pointer instead of an IPC handle. */
int  b200_exchange_set_peer(b200_runner *r, uint32_t peer_rank, void *device_ptr);
int  b200_exchange_configure(b200_runner *r, uint32_t rank, uint32_t world);
/* Sharded models, "deliver at emission" schedule (no reference counterpart: the reference does not shard a
 * model).  The thread that makes a neuron spike delivers that neuron's synapses of dendritic delay 0 and
 * 1 itself, into the rings of whichever process holds the target; so every process needs those synapses
 * of ITS neurons onto every process's neurons.  Each process builds them for all source neurons onto its
 * own targets (b200_near_export: 64-byte CUDA IPC handle + meta words 3 + 2 * neuron groups, meta[0] = 1
 * if the model qualifies), the caller all-gathers handle and meta, every process copies the rows of its
 * own neurons out of every process's table (b200_near_import, once per rank, itself included; common_shift[g] =
 * the largest meta[4 + 2 g] over all processes, 0xFFFFFFFF if the group is no spike source), the caller
 * synchronises the processes and every one calls b200_near_finish(agreed = all qualified).  Delay rings
 * must lie in the exchange arena.  All processes must then step in launches of the same lengths. */
int  b200_near_export(b200_runner *r, void *handle_64_bytes, uint64_t *meta, uint32_t meta_words);
int  b200_near_import(b200_runner *r, uint32_t peer_rank, const void *handle_64_bytes, const uint64_t *meta,
                      const uint32_t *common_shift);
int  b200_near_finish(b200_runner *r, int agreed);

/* ---- merged-group registration: pushMerged<Kind>Group<i>ToDevice
 *      (backendCUDAHIP.h:206-238, runtime.h:573-669) -------------------------- */
int  b200_push_neuron_update_group(b200_runner *r, uint32_t idx, const b200_neuron_group *g);
int  b200_push_synapse_group(b200_runner *r, uint32_t idx, const b200_synapse_group *g);
/* The checks b200_push_synapse_group applies, on their own (no runner, no GPU): missing arrays for the
 * connectivity / weight update model, a ring depth without d / den_delay, dendritic delay on BITMASK or
 * DENSE, pointers the vector loads cannot take (g 16-byte, ind four indices, d 4-byte aligned), delays
 * longer than the spike queues.  A descriptor that fails is never handed to a kernel. */
int  b200_validate_synapse_group(const b200_synapse_group *g);
int  b200_push_custom_update(b200_runner *r, const char *name, uint32_t idx, const b200_custom_update_group *u);

/* ---- initialisation kernels (backendSIMT.cc:1368-1779) --------------------- */
int  b200_initialize(b200_runner *r);
int  b200_initialize_sparse(b200_runner *r);
int  b200_init_var(b200_runner *r, void *device_ptr, uint32_t elem_bytes, uint64_t count,
                   uint32_t snippet, const float *params, uint32_t rng_stream);
int  b200_init_sparse_connectivity(b200_runner *r, uint32_t snippet, const float *params,
                                   uint32_t num_src, uint32_t num_trg, uint32_t row_stride,
                                   uint32_t ind_bytes, uint32_t trg_begin, uint32_t trg_end,
                                   uint32_t *row_length, void *ind, uint32_t rng_stream);
int  b200_init_sparse_vars(b200_runner *r, const uint32_t *row_length, uint32_t num_src,
                           uint32_t row_stride, void *device_ptr, uint32_t elem_bytes,
                           uint32_t snippet, const float *params, uint32_t rng_stream);
int  b200_build_remap(b200_runner *r, const uint32_t *row_length, const void *ind, uint32_t ind_bytes,
                      uint32_t num_src, uint32_t num_trg, uint32_t row_stride, uint32_t col_stride,
                      uint32_t *col_length, uint32_t *remap);

/* ---- the time step: stepTime / updateSynapses / updateNeurons
 *      (generateRunner.cc:270-299, backendCUDAHIP.cc:386-420, 548-589) ------- */
int  b200_update_synapses(b200_runner *r);
int  b200_update_neurons(b200_runner *r, uint64_t num_recording_timesteps);
int  b200_step_time(b200_runner *r, uint64_t num_steps, uint64_t num_recording_timesteps);
int  b200_custom_update(b200_runner *r, const char *name);
/* Data-parallel runs (every process holds a share of the batch; the reference: enableNCCLReductions,
 * backendCUDAHIP.cc:805-824, with ncclGenerateUniqueID / ncclGetUniqueID / ncclInitCommunicator exported by the
 * generated library, backends/cuda/backend.cc:219-226): one process obtains an id, the host application hands
 * it to every process, each creates its communicator.  From then on b200_custom_update reduces this process's
 * share, combines the reduced values of ALL updates of the group over the processes with one all-reduce per
 * operation (sum, max) on a packed buffer, and writes the combined value back, everything on the runner's
 * stream.  NCCL is loaded when first needed (the copy already in the process, else libnccl.so.2). */
int  b200_nccl_unique_id(void *id_128_bytes);
int  b200_nccl_init(b200_runner *r, const void *id_128_bytes, uint32_t rank, uint32_t world);
/* The two halves on their own (reduce this process's share into the targets; write the targets back),
 * for a host application that combines the targets itself. */
int  b200_custom_update_reduce(b200_runner *r, const char *name);
int  b200_custom_update_broadcast(b200_runner *r, const char *name);
/* Same, bracketed by CUDA events recorded on the runner's stream; waits for completion. */
int  b200_step_time_timed(b200_runner *r, uint64_t num_steps, uint64_t num_recording_timesteps, float *milliseconds);
/* A CUDA event pair on the runner's stream around whatever the caller enqueues in between (steps, custom
 * updates): begin waits for the stream and records, end records, waits and returns the elapsed time. */
int  b200_timed_begin(b200_runner *r);
int  b200_timed_end(b200_runner *r, float *milliseconds);
/* Waits for the stream and reports failed device-side checks (out-of-range index, row overflow, a wait inside a
 * persistent kernel that ran out).  After a wait that ran out the launch has ended early: the model's state is that
 * of an unknown step and, in a sharded model, words of the step may still be under way between the processes, so
 * the runner is to be destroyed (on every process of a sharded model); the CUDA context stays usable. */
int  b200_synchronize(b200_runner *r);
int  b200_get_timestep(b200_runner *r, uint64_t *timestep);
int  b200_set_timestep(b200_runner *r, uint64_t timestep);
int  b200_get_steps_done(b200_runner *r, uint64_t *steps);
/* Device-side counters: "synaptic_events" and "spikes" (when option count_events is on), "timestep", "steps_done".
 * Host-side answers: "lag_eligible" (1 if every SPARSE group has a dendritic-delay ring and no synapse with
 * delay 0, so spikes may be delivered one step late; scans the delay arrays if they changed), "lag" (1 if the
 * next persistent launch will do so). */
int  b200_get_counter(b200_runner *r, const char *name, uint64_t *value);
/* Tuning knobs (the counterpart of the backend Preferences, backends/cuda/backend.h:64-115):
 * "spike_lanes" (grid.y of the SPARSE kernel), "use_graph", "graph_steps", "count_events",
 * "use_fused" (persistent kernels),
 * "fused_blocks_per_sm", "fused_profile",
 * "use_lag" (default 1: when no synapse has dendritic delay 0 the persistent kernel delivers each spike one
 * step later into the ring slot one nearer, same result, one grid barrier per step instead of two),
 * "lag_agreed" (sharded model: the caller has checked "lag_eligible" on EVERY process; without it a sharded
 * model keeps the two-barrier schedule), "rescan_delays" (delay arrays were changed by something other than
 * this library's push / init calls), "use_near_queues" (default 1: a sharded model on the
 * "deliver at emission" schedule sends near synapses between processes through per-CTA queues of self-validating
 * words; 0: reduces them straight into the other process's rings and fences) / "near_queue_words" (capacity of
 * one queue, 2 .. 2048; what does not fit goes the direct way), "use_tiled" / "tiled_min_events" (target-tiled SPARSE delivery of steps
 * with at least that many estimated events on the one-launch-per-kernel path; 0: every step.  The tiled kernels
 * are launched only while the largest spike count of the steps before says such a step may come: counter
 * "tiled_armed"; b200_update_synapses always launches them), "tiled_ticket_events" / "tiled_ticket_cost" (the
 * tiled kernel's unit of work, handed to one warp, is sized for about that many synaptic events, default 2048;
 * its fixed cost in synaptic events when a step's work is cut into equal stretches per CTA, default 256),
 * "barrier_spin_limit" / "exchange_spin_limit" (polls) and "stream_wait_cycles" (SM cycles): how long a wait
 * inside a persistent kernel lasts before the launch gives up and b200_synchronize reports
 * B200_ERR_DEVICE_CHECK (defaults: tens of milliseconds; about two seconds). */
int  b200_set_option(b200_runner *r, const char *name, double value);

/* Which time-step path b200_step_time takes for the registered model: 1 = persistent kernel (one
 * cooperative launch runs all the steps), 0 = one launch per kernel (CUDA graph).  `why` (may be NULL)
 * receives the reason the persistent kernel was not chosen. */
int  b200_get_step_path(b200_runner *r, int *path, char *why, size_t why_bytes);

/* ---- timers: neuronUpdateTime etc. (generateRunner.cc:159-222) ------------- */
int  b200_enable_timing(b200_runner *r, int enabled);
int  b200_get_timer(b200_runner *r, const char *name, double *seconds);
int  b200_reset_timers(b200_runner *r);
int  b200_get_kernel_launches(b200_runner *r, uint64_t *launches);
/* SM cycles thread 0 of every CTA of the persistent kernel spent in {presynaptic work, barrier,
 * neuron work, barrier}, accumulated while option "fused_profile" is on: out[cta*4 + phase]. */
int  b200_get_cta_cycles(b200_runner *r, uint64_t *out, uint32_t max_ctas, uint32_t *num_ctas);

/* ---- neuron update without any allocation ------------------------------------
 * No counterpart in the reference, whose runtime allocates every array and every
 * merged-group table itself (runtime.cc:147-662).
 *
 * Performs what b200_push_neuron_update_group + b200_update_neurons perform for
 * one time step, for callers that may not allocate while they run: hard
 * real-time loops (an allocator call has unbounded latency and can synchronise
 * the device) and plugins inside a process with a fixed memory budget.  The
 * descriptor tables, block lookup table and step counters
 * that the regular path keeps in cudaMalloc'ed memory live in a fixed array
 * inside the library image instead (B200_NOALLOC_SCRATCH_BYTES on every GPU that
 * loads the library, for the life of the process), which caps the call at
 * B200_NOALLOC_MAX_GROUPS neuron groups; more is rejected with B200_ERR_INVALID.
 * `groups` is a HOST array of descriptors holding the caller's device pointers;
 * `stream` is a cudaStream_t (NULL for the default stream); `timestep` and
 * `steps_done` are the values the regular path would hold on the device.
 * The first call on a device resolves the array's address and should be made
 * before any stream capture begins.  A call on a stream that is being captured
 * is refused with B200_ERR_STATE: every call copies its tables and counters from
 * host memory that no longer exists when a graph would replay.  Calls on one
 * device share the array: calls whose GPU work may overlap must be ordered by
 * the caller.  No host or device memory is allocated or freed, and the caller's
 * current device is restored before returning.  Errors: b200_noalloc_last_error().
 *
 * b200_noalloc_check waits for `stream` and returns B200_ERR_DEVICE_CHECK if the
 * last update on that device failed a kernel-side bounds check (more spikes in
 * a step than the spike list holds: the surplus spikes were dropped); it
 * allocates nothing either.  The next update clears the condition. */
#define B200_NOALLOC_MAX_GROUPS     64
#define B200_NOALLOC_SCRATCH_BYTES  40960
int  b200_update_neurons_noalloc(int device, void *stream, const b200_neuron_group *groups, uint32_t num_groups,
                                 uint32_t batch_size, double dt, uint64_t seed, uint64_t timestep,
                                 uint64_t steps_done, uint64_t num_recording_timesteps);
int  b200_noalloc_check(int device, void *stream);
const char *b200_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* GENN_B200_H */
