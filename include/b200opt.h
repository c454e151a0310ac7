/*
 * b200opt — C ABI of the B200-native replacement for Saga's data-parallel
 * parameter update: gradient reduce-scatter across GPUs, mixed-precision Adam
 * with overflow detection and unscale on the locally owned shard, and the
 * all-gather of the updated weights, run as ONE fused sm_100a kernel per rank
 * that reads and writes peer GPU memory directly over NVLink.
 *
 * Everything here is plain C: opaque handles, raw device/host pointers, sizes
 * and status codes.  No exception and no abort crosses this boundary.
 *
 * Paths in "replaces" notes are relative to the Saga project root.
 *
 * Threading: b200opt_step / b200opt_step_host / b200opt_flags may be called
 * concurrently from different host threads as long as each thread uses a
 * different handle (one handle == one rank == one GPU), which is how Saga
 * drives its contexts (one std::thread per GPU, test/test_classifier.cpp:689).
 * Creation, wiring and destruction are not thread-safe.
 */
#ifndef B200OPT_H
#define B200OPT_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define B200OPT_API __attribute__((visibility("default")))
#else
#define B200OPT_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define B200OPT_MAX_RANKS 8

/* status codes */
#define B200OPT_OK 0
#define B200OPT_EINVAL (-1)       /* bad argument */
#define B200OPT_ECUDA (-2)        /* a CUDA runtime call failed; see b200opt_last_error */
#define B200OPT_ENOMEM (-3)       /* device or host allocation failed */
#define B200OPT_ETIMEOUT (-4)     /* a peer rank did not arrive within the wait limit */
#define B200OPT_ESTATE (-5)       /* call not valid in the handle's state (peers not wired, ...) */
#define B200OPT_EUNSUPPORTED (-6) /* built without the needed support (e.g. NCCL) */
#define B200OPT_ETOOBIG (-7)      /* size beyond what the fixed scratch of an entry point covers */

/* dtype groups, the two the reference builds optimizers for
 * (src/cuda/cuda_optimizer.cpp:276-292) */
#define B200OPT_HALF 0
#define B200OPT_FLOAT 1

/* loss-scale policies for b200opt_policy_update */
#define B200OPT_POLICY_REFERENCE 0 /* src/cuda/cuda_program.cpp:295-302 */
#define B200OPT_POLICY_INTERVAL 1  /* halve on inf/nan, double after N clean steps */

/* collective paths for b200opt_set_option(B200OPT_OPT_PATH) */
#define B200OPT_PATH_AUTO 0 /* peer kernel; NCCL below the measured crossover or when the
                               GPUs cannot reach one another's memory */
#define B200OPT_PATH_PEER 1 /* fused peer-memory kernel always: gradients summed in rank
                               order, bit for bit reproducible */
#define B200OPT_PATH_NCCL 2 /* ncclReduceScatter + Adam kernel + ncclAllGather */
#define B200OPT_PATH_NVLS 3 /* fused kernel over an NVSwitch multicast mapping: the switch
                               sums the fp16 gradients (its own arithmetic: within one fp16
                               ulp of the correctly rounded sum, the same NCCL's NVLS
                               reduce-scatter has) and replicates the weights; needs
                               B200OPT_CREATE_MULTICAST */

/* options */
#define B200OPT_OPT_TIMEOUT_MS 1    /* limit of every cross-GPU wait (default 10000) */
#define B200OPT_OPT_PATH 2          /* B200OPT_PATH_* */
#define B200OPT_OPT_CTAS_PER_SM 3   /* launch shape of the fused kernel (tuning) */
#define B200OPT_OPT_KERNEL_VARIANT 4 /* 0 = default of the rank count; 1 = direct 16-byte loads; 2 = bulk-copy staging through shared memory */
#define B200OPT_OPT_NCCL_CROSSOVER 5 /* AUTO uses NCCL when n_half is below this many elements */
#define B200OPT_OPT_STAGES 6        /* depth of the shared-memory ring of the staged kernel (tuning) */
#define B200OPT_OPT_GRID 7          /* number of CTAs of the step kernel, overrides CTAS_PER_SM (tuning) */
#define B200OPT_OPT_PHASE_TIMERS 8  /* 1: the step kernel records where its time went (b200opt_phase_times) */
#define B200OPT_OPT_ASSUME_NO_PEER_ACCESS 9 /* test aid, set before wiring: treat every other GPU as
                                               unreachable, as on a machine without peer access */

#define B200OPT_OPT_KEEP_REDUCED 10 /* multicast path: 1 leaves the switch-reduced gradients of the own
                                       shard in the own gradient buffer (where ncclReduceScatter leaves
                                       them in place in the reference), so that a caller can check the
                                       update against the sum it was computed from */

/* creation flags for b200opt_create_ex / b200opt_create_group_ex */
#define B200OPT_CREATE_FABRIC 1u    /* weight/gradient arena from CUDA's virtual-memory API: shared
                                       between processes as a file descriptor (b200opt_fd_export),
                                       not as a CUDA IPC handle */
#define B200OPT_CREATE_MULTICAST 2u /* implies FABRIC; b200opt_create_group_ex also binds the arenas
                                       of all ranks to one NVSwitch multicast object
                                       (B200OPT_EUNSUPPORTED where the GPUs cannot) */

typedef struct b200opt b200opt_t;

/* ------------------------------------------------------------------ version */

/* Returns a static string such as "b200opt 0.1 sm_100a". */
B200OPT_API const char *b200opt_version(void);

/* Human-readable text for a status code. */
B200OPT_API const char *b200opt_strerror(int status);

/* Text of the last failure recorded on this handle ("" if none). */
B200OPT_API const char *b200opt_last_error(const b200opt_t *h);

/* ----------------------------------------------------------------- creation */

/*
 * Creates rank `rank` of `nranks` on CUDA device `device`, owning
 *   - the flat weight and gradient buffers of both dtype groups
 *     (n_half fp16 elements and n_float fp32 elements each, zero-filled), and
 *   - the shard-sized Adam state m, v (and the fp32 master copy for the fp16
 *     group), zero-filled.
 * Replaces the allocation half of CudaProgram::create_optimizer
 * (src/cuda/cuda_optimizer.cpp:221-229: one [weights | gradients] allocation
 * per dtype) and the AdamF32 / AdamMixed constructors (:64-74, :122-146).
 * The shard of rank r is elements [r*(n/nranks), (r+1)*(n/nranks)) of each
 * flat buffer, the reference's partition (:85-86, :157-158); elements beyond
 * nranks*(n/nranks) are never updated, as in the reference.
 * Either count may be 0.  nranks <= B200OPT_MAX_RANKS.
 * With nranks > 1 the peers must be wired (below) before the first step.
 */
B200OPT_API int b200opt_create(b200opt_t **out, int rank, int nranks, int device,
                   size_t n_half, size_t n_float);
/* The same with B200OPT_CREATE_* flags (0 = b200opt_create). */
B200OPT_API int b200opt_create_ex(b200opt_t **out, int rank, int nranks, int device,
                      size_t n_half, size_t n_float, unsigned flags);

/*
 * Single-process convenience: creates all ranks and wires them to one another,
 * the counterpart of CudaEngine::createContexts(multi=true) +
 * ncclCommInitAll (src/cuda/cuda_common.cpp:89-129).  devices[i] is the CUDA
 * device of rank i.  When several ranks name the SAME device the group runs in
 * serial mode: kernels of different ranks never wait for one another (they
 * could not run concurrently on one GPU); instead the caller must have written
 * every rank's gradients before stepping any rank, must step every rank, and
 * reads flags only after all ranks stepped.  Serial mode exists so that the
 * multi-rank arithmetic can be checked on a single GPU.
 */
B200OPT_API int b200opt_create_group(b200opt_t **out, int nranks, const int *devices,
                         size_t n_half, size_t n_float);
B200OPT_API int b200opt_create_group_ex(b200opt_t **out, int nranks, const int *devices,
                            size_t n_half, size_t n_float, unsigned flags);

/* Frees everything the handle owns.  Streams belong to the caller.  Ranks that
 * share a multicast object must all have finished stepping (a host barrier
 * between the last b200opt_flags and the first b200opt_destroy) before any of
 * them is destroyed: a rank must never issue a multicast access to memory
 * another rank has already unbound. */
B200OPT_API int b200opt_destroy(b200opt_t *h);

/* ------------------------------------------------------------- peer wiring */

/*
 * One rank per process (torchrun-style launch): every rank exports 64 bytes,
 * the launcher exchanges them (any host transport), and every rank attaches
 * every other rank's bytes.  Replaces the role of ncclCommInitAll
 * (src/cuda/cuda_common.cpp:116-127).
 */
#define B200OPT_IPC_HANDLE_BYTES 64
B200OPT_API int b200opt_ipc_export(b200opt_t *h, void *handle_out);
B200OPT_API int b200opt_ipc_attach(b200opt_t *h, int peer_rank, const void *handle);

/* Same process, other rank's handle (what b200opt_create_group does).  When
 * the two GPUs have no peer access the peer is recorded as unreachable instead
 * of failing: B200OPT_PATH_AUTO then steps through NCCL (b200opt_nccl_init),
 * the fallback the reference's own path is (src/cuda/cuda_optimizer.cpp:160-185). */
B200OPT_API int b200opt_attach_local(b200opt_t *h, int peer_rank, b200opt_t *peer);

/*
 * Wiring of handles created with B200OPT_CREATE_FABRIC, one rank per process:
 * every rank exports a file descriptor of its arena, the launcher passes it to
 * every other process (SCM_RIGHTS over a Unix socket) and closes it; every
 * rank attaches the descriptors it received.  Then, for the multicast path:
 * rank 0 calls b200opt_mc_create and the launcher passes that descriptor to
 * the other ranks, which call b200opt_mc_join; after EVERY rank has returned
 * from create/join (a host barrier) every rank calls b200opt_mc_bind.  No
 * counterpart in the reference, whose collectives are NCCL's.
 */
B200OPT_API int b200opt_fd_export(b200opt_t *h, int *fd);
B200OPT_API int b200opt_fd_attach(b200opt_t *h, int peer_rank, int fd);
B200OPT_API int b200opt_multicast_supported(int device, int *yes);
B200OPT_API int b200opt_mc_create(b200opt_t *h, int *fd);
B200OPT_API int b200opt_mc_join(b200opt_t *h, int fd);
B200OPT_API int b200opt_mc_bind(b200opt_t *h);

/*
 * Optional NCCL communicator for the fallback path.  `unique_id` is the 128
 * bytes of an ncclUniqueId that rank 0 obtained from
 * b200opt_nccl_unique_id and the launcher distributed.
 */
#define B200OPT_NCCL_ID_BYTES 128
B200OPT_API int b200opt_nccl_unique_id(void *unique_id_out);
B200OPT_API int b200opt_nccl_init(b200opt_t *h, const void *unique_id);

/* ------------------------------------------------------------------ buffers */

/*
 * Device pointers of this rank's flat weight and gradient buffers of one dtype
 * group and their element count, so that the caller can point its tensors into
 * them exactly as create_optimizer re-points Saga's tensor storages
 * (src/cuda/cuda_optimizer.cpp:245-249).  Valid until b200opt_destroy.
 */
B200OPT_API int b200opt_buffers(b200opt_t *h, int dtype, void **weights, void **gradients,
                    size_t *n);

/*
 * The reference's flat layout: tensor j starts at the sum of the sizes before
 * it, each rounded up to a multiple of 16 elements
 * (src/cuda/cuda_optimizer.cpp:199-219,235-258).  Writes k offsets (may be
 * NULL) and returns the padded total through *total.  Host-only.
 */
B200OPT_API int b200opt_layout(const size_t *sizes, size_t k, size_t *offsets,
                   size_t *total);

/*
 * After the initial weights have been written into the weight buffers:
 * master := float(fp16 weight) over this rank's shard, m = v = 0, iteration
 * counter = 0.  Replaces the host loop of the AdamMixed constructor
 * (src/cuda/cuda_optimizer.cpp:142-145).  Asynchronous on `stream`.
 */
B200OPT_API int b200opt_init_master(b200opt_t *h, void *stream);

/* --------------------------------------------------------------------- step */

/*
 * One optimizer step for both dtype groups of this rank, enqueued on `stream`
 * (a cudaStream_t) and asynchronous: replaces AdamF32::exec + AdamMixed::exec
 * (src/cuda/cuda_optimizer.cpp:76-113,148-186) and the 12-byte flag all-reduce
 * of CudaProgram::step (src/cuda/cuda_program.cpp:282-291).
 *   lr, l2_lambda  ProgramConfig::learning_rate / l2_lambda (saga.hpp:500-503)
 *   scale          the program's current loss scale (m_mp_scaling); the fp16
 *                  group's gradients are multiplied by 1.0f/scale
 * The iteration counter advances on every call, overflow or not.
 * All ranks must call it the same number of times; with nranks > 1 the kernel
 * waits (bounded) for every peer's call of the same step.
 */
B200OPT_API int b200opt_step(b200opt_t *h, float lr, float l2_lambda, float scale,
                 void *stream);

/*
 * One step issued as several buckets, so that the reduction and update of the
 * gradients that backward has already finished can run (on a stream of the
 * caller's choosing) while backward is still producing the others.  The
 * reference can only start after ALL backward ops: its optimizer ops are
 * appended behind them (src/cuda/cuda_program.cpp:455).
 *   b200opt_step_begin   opens the step: advances the iteration counter once
 *   b200opt_step_bucket  the fused reduce + update + gather for elements
 *                        [first, first+count) of each dtype group's flat buffer
 *                        (each rank does the part that lies in its shard).
 *                        Every element must be covered by exactly one bucket
 *                        of the step; every rank issues the same buckets in the
 *                        same order; `last` != 0 marks the final bucket, whose
 *                        kernel also completes the step across ranks (flag
 *                        sums, all weights landed).  b200opt_flags after it.
 * Buckets of one step give bit for bit the result of one b200opt_step.  With
 * several ranks each bucket's kernel waits (bounded) until every rank has
 * issued the same bucket, i.e. until that bucket's gradients are final
 * everywhere.  The kernel then OVERWRITES the bucket's weights in every
 * rank's weight buffer, without a further barrier for any but the last
 * bucket.  A bucket may therefore be issued only behind every backward op
 * that WRITES its gradients AND every backward op that still READS its
 * weights (a layer's data-gradient op reads the layer's weights), on this
 * rank's stream; the cross-rank wait then extends that guarantee to all ranks.
 * A refused bucket moves no counter and leaves the step open.  Not available
 * on the NCCL path.
 */
B200OPT_API int b200opt_step_begin(b200opt_t *h);
B200OPT_API int b200opt_step_bucket(b200opt_t *h, size_t half_first,
                                    size_t half_count, size_t float_first,
                                    size_t float_count, float lr,
                                    float l2_lambda, float scale, void *stream,
                                    int last);

/*
 * Same step, gradients taken from HOST memory: copies grads_half (n_half fp16)
 * and grads_float (n_float fp32) into the gradient buffers on `stream`, steps,
 * waits for the stream and returns the flag sums.  Either pointer may be NULL
 * when its group is empty.  Pinned host memory makes the copies asynchronous.
 * On one rank, from 2^22 fp16 elements up, the copy is cut into eight chunks
 * on a stream of the library's own and the step is issued as one bucket per
 * chunk behind it (b200opt_step_bucket), so that the update overlaps the
 * transfer; the result is bit for bit that of one whole step.  The first such
 * call creates that stream and its events.
 */
B200OPT_API int b200opt_step_host(b200opt_t *h, const void *grads_half,
                      const void *grads_float, float lr, float l2_lambda,
                      float scale, void *stream, uint32_t flags_out[3]);

/*
 * Loss scale resident on the device: removes the per-step host synchronise
 * that CudaProgram::step needs to read the flags and update m_mp_scaling
 * (src/cuda/cuda_program.cpp:293-302).  After b200opt_device_scale_enable the
 * scale lives in this rank's control page; b200opt_step_device_scale takes
 * 1/scale from there and the step kernel's last CTA applies the policy (same
 * float-state, double-factor arithmetic) to it once the flag sums are known,
 * so steps can be enqueued back to back without the host in the loop.  Every
 * rank computes the same scale from the same sums.
 *   b200opt_device_scale_ptr   device address of the live scale, for the
 *                              kernels that multiply the loss gradient by it
 *                              (src/cuda/cuda_dnn.cpp:1315,1428-1443 pass it
 *                              by value today)
 *   b200opt_device_scale_read  waits for `stream`; returns the current scale
 *                              and the log of the last `log_capacity` steps,
 *                              oldest first, four words per step:
 *                              {range, inf, nan, bits of the scale after it}
 *   b200opt_device_scale_peek  does not wait and makes no CUDA call: the scale
 *                              after the last step whose kernel has FINISHED
 *                              (the kernel leaves it in the pinned result
 *                              page) and that step's number; the initial
 *                              scale and 0 before any step has finished.  For
 *                              a host that paces itself with events one step
 *                              behind the device and wants a scale to show
 *                              (the UI cell of src/cuda/cuda_program.cpp:316)
 *                              without draining the stream.
 * Not available in serial mode or on the NCCL path.
 */
B200OPT_API int b200opt_device_scale_enable(b200opt_t *h, float initial_scale,
                                            int policy, int interval,
                                            size_t log_capacity);
B200OPT_API int b200opt_device_scale_ptr(b200opt_t *h, const float **scale_dev);
B200OPT_API int b200opt_step_device_scale(b200opt_t *h, float lr,
                                          float l2_lambda, void *stream);
B200OPT_API int b200opt_device_scale_read(b200opt_t *h, void *stream,
                                          float *scale, uint32_t *log_out,
                                          size_t capacity, size_t *count);
B200OPT_API int b200opt_device_scale_peek(b200opt_t *h, float *scale,
                                          uint32_t *step);

/*
 * Waits for `stream`, then returns the sums over ranks of {range, inf, nan}
 * raised by the last step and clears them: the values CudaProgram::step reads
 * from m_aux after its stream synchronise (src/cuda/cuda_program.cpp:293-306).
 * Returns B200OPT_ETIMEOUT if a cross-GPU wait of that step ran out; the
 * handle then refuses further steps.
 */
B200OPT_API int b200opt_flags(b200opt_t *h, void *stream, uint32_t flags_out[3]);

/*
 * The loss-scale update of CudaProgram::step (src/cuda/cuda_program.cpp:295-302),
 * bit for bit: scale is a float, the factors are double.
 *   B200OPT_POLICY_REFERENCE: inf or nan -> x0.5; else range > 1 -> x0.9; else x1.02
 *   B200OPT_POLICY_INTERVAL:  inf or nan -> x0.5 and *state = 0; else
 *                             ++*state == interval -> x2.0 and *state = 0
 * `state` and `interval` are ignored by the reference policy.  Host-only.
 */
B200OPT_API int b200opt_policy_update(float *scale, const uint32_t flags[3], int policy,
                          int *state, int interval);

/* The two scalars AdamMixed::exec derives per step
 * (src/cuda/cuda_optimizer.cpp:150-152): 1/(1-0.9^iter), 1/(1-0.999^iter),
 * computed in double and narrowed to float.  Host-only. */
B200OPT_API int b200opt_bias_corrections(int iter, float *b1t, float *b2t);

/*
 * The rule by which a step picks its collective path (B200OPT_PATH_*), from
 * the requested path and what the group has: several ranks stepped serially
 * on one GPU, peers' memory reachable, an NCCL communicator, a bound multicast
 * object.  Returns B200OPT_ESTATE when the requested path lacks its
 * communicator or multicast object, B200OPT_EUNSUPPORTED when no path is
 * usable.  Host-only; b200opt_step applies it before it moves any counter.
 */
B200OPT_API int b200opt_choose_path(int requested, int nranks, int serial,
                        int peers_reachable, int have_nccl, int have_multicast,
                        size_t n_half, size_t nccl_crossover, int *chosen);

/* ------------------------------------------------------------ kernel seam */

/*
 * Drop-in for saga::adam_mixed (src/cuda/cuda_kernels.hpp:61-64,
 * src/cuda/cuda_kernels.cu:241-250) on caller-owned device memory, one GPU, no
 * collective.  `aux` points at device-accessible {range, inf, nan, anomaly}
 * words (src/cuda/cuda_aux.hpp:5-10); flags seen are stored as 1.
 * Any pointer alignment is accepted; 16-byte aligned pointers take the
 * vectorised path.
 */
B200OPT_API int b200opt_adam_mixed(size_t n, float alpha, void *weights,
                       const void *gradients, float *mvec, float *vvec,
                       float *cvec, float b1t, float b2t, float learning_rate,
                       float l2_lambda, uint32_t *aux, void *stream);

/* Drop-in for saga::adam_float (src/cuda/cuda_kernels.hpp:57-59,
 * src/cuda/cuda_kernels.cu:232-239). */
B200OPT_API int b200opt_adam_float(size_t n, float *weights, const float *gradients,
                       float *mvec, float *vvec, float b1t, float b2t,
                       float learning_rate, float l2_lambda, uint32_t *aux,
                       void *stream);

/*
 * No counterpart in the reference: the same one-GPU mixed-precision Adam step
 * as b200opt_adam_mixed for callers that must not allocate device memory.
 *
 * Who that is: a program whose device memory is planned once up front (Saga
 * itself lays every tensor out in one arena before the first step and never
 * allocates again), a step loop that cannot tolerate the device-wide
 * synchronisation an allocation or free may imply, or an embedder running under
 * a fixed memory reservation.  The handle API above needs cudaMalloc for its
 * control block; this entry point needs none.  The kernel's scratch (the
 * counter and flag words its CTAs meet on) lives in a fixed
 * B200OPT_STATIC_SCRATCH_BYTES array inside the library image, which every GPU
 * that loads the library holds until the process exits.  Nothing in this call
 * allocates or frees memory, on the device or through any library.
 *
 *   - Inputs and outputs are the caller's: weights/gradients (fp16), mvec, vvec,
 *     cvec (fp32), all n elements and 16-byte aligned, and flags_out, three
 *     u32 in device memory which receive {range, inf, nan} as 0 or 1
 *     (overwritten, not accumulated).
 *   - n may not exceed B200OPT_STATIC_MAX_ELEMS; larger sizes return
 *     B200OPT_ETOOBIG and launch nothing.
 *   - The first call on a device looks up the array's device address and
 *     raises the kernel's dynamic shared-memory limit (cudaFuncSetAttribute);
 *     make that first call during start-up, before any stream capture is open.
 *   - The kernel's waits on its own asynchronous copies are bounded (10 s).  If
 *     one ever ran out, the kernel stops early and this entry point reports it
 *     by writing 0xFFFFFFFF into all three flag words; m, v, master and weights
 *     are then partly updated.
 *   - All calls on one GPU share the array and it keeps what the last call left:
 *     each call clears the words that must start at zero on `stream` before its
 *     kernel.  Two calls that overlap on the same GPU (different streams, or
 *     different host threads) race on it and give undefined flags; serialise
 *     them on one stream.
 */
#define B200OPT_STATIC_SCRATCH_BYTES 4096
#define B200OPT_STATIC_MAX_ELEMS ((size_t)1 << 30)
B200OPT_API int b200opt_adam_mixed_static(size_t n, float alpha, void *weights,
                                          const void *gradients, float *mvec,
                                          float *vvec, float *cvec, float b1t,
                                          float b2t, float learning_rate,
                                          float l2_lambda, uint32_t *flags_out,
                                          void *stream);

/* ------------------------------------------------------- state and options */

/* Iteration counter (AdamMixed::m_iter, src/cuda/cuda_optimizer.cpp:41). */
B200OPT_API int b200opt_get_iter(const b200opt_t *h, int *iter);
B200OPT_API int b200opt_set_iter(b200opt_t *h, int iter);

/*
 * Copies this rank's shard state to / from host memory (synchronous):
 * which = 0 m, 1 v, 2 master (fp16 group only).  count receives / gives the
 * shard length n/nranks.  The reference never saves this state
 * (src/graph.cpp:60-104 saves weights only); these make an exact resume
 * possible.
 */
B200OPT_API int b200opt_export_state(b200opt_t *h, int dtype, int which, float *host_dst,
                         size_t capacity, size_t *count);
B200OPT_API int b200opt_import_state(b200opt_t *h, int dtype, int which,
                         const float *host_src, size_t count);

/* This handle's rank and the number of ranks it was created for. */
B200OPT_API int b200opt_rank_info(const b200opt_t *h, int *rank, int *nranks);

/*
 * One tensor in Saga's own file format (Tensor::save / Tensor::load,
 * src/tensor.cpp:1382-1552): 8 bytes "sagaT001", u32 element type (0 float,
 * 1 half), u32 rank (<= 8), rank x u32 dimensions, the elements in row-major
 * order; written to "<path>.tmp" and renamed into place.  dtype is
 * B200OPT_HALF or B200OPT_FLOAT.  b200opt_tensor_load fills whichever outputs
 * are non-NULL; with data == NULL it only reads the header and reports the
 * payload size through *bytes.  Host-only.
 */
B200OPT_API int b200opt_tensor_save(const char *path, int dtype, unsigned rank,
                        const uint32_t *dims, const void *data);
B200OPT_API int b200opt_tensor_load(const char *path, int *dtype, unsigned *rank,
                        uint32_t dims[8], void *data, size_t capacity_bytes,
                        size_t *bytes);

/*
 * Optimizer-state checkpoint of this rank in directory `dir` (which must
 * exist), as Saga tensor files: adam.r<rank>of<nranks>.{half.m, half.v,
 * half.master, float.m, float.v, meta}.saga.  The shard arrays are fp32
 * vectors; "meta" holds the iteration counter, the loss scale passed in and
 * the policy's clean-step count.  Saga's own Graph save keeps the weights
 * (src/graph.cpp:60-104) and nothing else; with these files a resumed run
 * continues bit for bit.  Loading refuses files written for another rank,
 * rank count or buffer size.  Synchronous; call between steps.
 */
B200OPT_API int b200opt_checkpoint_save(b200opt_t *h, const char *dir, float scale,
                            int policy_state);
B200OPT_API int b200opt_checkpoint_load(b200opt_t *h, const char *dir, float *scale,
                            int *policy_state);

B200OPT_API int b200opt_set_option(b200opt_t *h, int option, long value);
B200OPT_API int b200opt_get_option(const b200opt_t *h, int option, long *value);

/*
 * With B200OPT_OPT_PHASE_TIMERS set: where the last step kernel of this rank
 * spent its time, nanoseconds of the GPU's global timer, valid after
 * b200opt_flags:
 *   [0] wait for every rank's "gradients final" announcement (first CTA)
 *   [1] kernel entry until the last CTA finished its share of the shard
 *   [2] completion protocol in the last CTA (flag exchange, wait until every
 *       rank has finished reading gradients and writing weights)
 *   [3] kernel entry until the end of the completion protocol
 */
B200OPT_API int b200opt_phase_times(const b200opt_t *h, uint64_t ns_out[4]);

/*
 * Measurement aid: copies the first `bytes` of the peer rank's fp16 weight
 * buffer over this rank's, on `stream`, with the GPU's copy engines.  After
 * any completed step all ranks hold the same weights, so the copy changes
 * nothing; it lets a benchmark measure the NVLink copy rate between the very
 * arenas the step kernel uses.  No counterpart in the reference.
 */
B200OPT_API int b200opt_peer_copy(b200opt_t *h, int peer_rank, size_t bytes, void *stream);

/* Kernel launches this handle has issued since creation (its own kernels and,
 * on the NCCL path, the NCCL calls). */
B200OPT_API int b200opt_launch_count(const b200opt_t *h, uint64_t *launches);

#ifdef __cplusplus
}
#endif
#endif /* B200OPT_H */
