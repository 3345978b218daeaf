/* C ABI of the B200 configurable hierarchical collectives library.
 *
 * Three layers are exported:
 *   1. step programs  (chb_program_*): compile an algorithm into a schedule,
 *      inspect / verify / simulate it on the host;
 *   2. communicators  (chb_comm_*): symmetric scratch + signal pads shared by
 *      the GPUs of one NVLink domain, or an emulated world on a single GPU;
 *   3. collectives    (chb_* / the reference-compatible *_radix_batch calls):
 *      launch sm_100a kernels on a stream.
 *
 * Every function returns CHB_SUCCESS (0) or a positive error code; functions
 * that can fail for several reasons also fill an optional message buffer.
 */
#ifndef CHB_H_
#define CHB_H_
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  CHB_SUCCESS = 0,
  CHB_ERR_NO_MEM = 1,   /* allocation failed                                  */
  CHB_ERR_OTHER = 2,
  CHB_ERR_COUNT = 3,    /* count not acceptable for this algorithm            */
  CHB_ERR_OP = 4,       /* reduction not supported for this dtype / algorithm */
  CHB_ERR_ARG = 5,      /* invalid argument (P % b != 0, unknown name, ...)   */
  CHB_ERR_TIMEOUT = 6,  /* a bounded device-side wait expired                 */
  CHB_ERR_CUDA = 7,
  CHB_ERR_UNSUPPORTED = 8
};

/* element types and reductions (same numbering as chb::DType / chb::RedOp) */
enum { CHB_F32 = 0, CHB_BF16 = 1, CHB_F16 = 2, CHB_I32 = 3, CHB_F64 = 4, CHB_I64 = 5, CHB_U8 = 6 };
enum { CHB_SUM = 0, CHB_MAX = 1, CHB_MIN = 2, CHB_PROD = 3 };

/* ------------------------------------------------------------------ programs */
typedef struct chb_program chb_program_t;

/* in_symmetric: bit 0 = peers may read the caller's input directly, bit 1 = the
 * input aliases the output (every read of the input goes through scratch). */
chb_program_t* chb_program_create(const char* coll, const char* algo, int P, int k, int b,
                                  int64_t count, int aux, int in_symmetric, int out_symmetric,
                                  char* err, int errlen);
/* all-to-all-v with the radix-r / batch-b store-and-forward routing; counts[s*P + d] = elements rank s
 * sends to rank d, blocks packed contiguously (input in destination order, output in source order) */
chb_program_t* chb_program_create_alltoallv(int P, int r, int b, const int64_t* counts, char* err, int errlen);
void chb_program_destroy(chb_program_t* p);

enum {
  CHB_INFO_P = 0, CHB_INFO_NROUNDS, CHB_INFO_IN_ELEMS, CHB_INFO_OUT_ELEMS, CHB_INFO_WORK_ELEMS,
  CHB_INFO_NOPS, CHB_INFO_REMOTE_MSGS, CHB_INFO_REMOTE_ELEMS, CHB_INFO_MAX_RANK_REMOTE_ELEMS,
  CHB_INFO_LOCAL_ELEMS, CHB_INFO_MAX_NSRC, CHB_INFO_READS_PEER_IN, CHB_INFO_READS_PEER_OUT,
  CHB_INFO_NSRCS, CHB_INFO_NWAITS, CHB_INFO_NEXIT_WAITS, CHB_INFO_NSIGNALS, CHB_INFO_COUNT_
};
int chb_program_info(const chb_program_t* p, int64_t* info, int n);
const char* chb_program_name(const chb_program_t* p);
/* number of hazards not covered by the program's own synchronisation (0 = ok) */
int chb_program_verify(const chb_program_t* p, char* err, int errlen);
/* run all ranks on host buffers; in[r] / out[r] are rank r's buffers */
int chb_program_simulate(const chb_program_t* p, int dtype, int op, void* const* in,
                         void* const* out, uint64_t seed, char* err, int errlen);
/* The push (flagged-line) form of a program, see sched/ll_plan.h.
 * chb_program_ll_lines: lines the fullest inbox needs for elements of esz bytes (-1: bad argument).
 * chb_program_ll_info: info = rounds, messages pushed in a round's push phase, messages forwarded line by line
 *   from the previous round's steps, rank-local barriers (summed over ranks), lines in the fullest inbox, lines
 *   of the busiest (rank, round), bytes of the largest rank's own table entries (what a CTA of the executor
 *   keeps in shared memory when it fits).
 * chb_program_simulate_ll: run that form on host buffers, line by line, nthreads virtual threads per rank
 *   advanced in a random order (seed); a message that nobody sends ends as CHB_ERR_TIMEOUT with the waiting
 *   rank and peer in err.  fault: 0, or a defect injected into the plan to test the simulator itself
 *   (1 = its barriers are ignored, 2 = the last forward of every step is left out).  launches: how often the
 *   program runs back to back, each rank going on as soon as its own previous launch has returned (the inbox
 *   halves alternate; a line overwritten before it was read ends the run with CHB_ERR_TIMEOUT). */
long long chb_program_ll_lines(const chb_program_t* p, int esz);
int chb_program_ll_info(const chb_program_t* p, int esz, long long* info, int n);
int chb_program_simulate_ll(const chb_program_t* p, int dtype, int op, void* const* in, void* const* out,
                            uint64_t seed, int nthreads, int fault, int launches, char* err, int errlen);
/* run all ranks as host threads (real concurrency); mean wall seconds per repetition in *seconds */
int chb_program_run_threads(const chb_program_t* p, int dtype, int op, void* const* in, void* const* out,
                            int iters, double* seconds);
/* the same, once, with rank late_rank entering delay_ms late; until it enters, its input holds poison
 * (checks that no peer reads a directly pulled input before its owner has entered the collective) */
int chb_program_run_threads_late(const chb_program_t* p, int dtype, int op, void* const* in, void* const* out,
                                 int late_rank, int delay_ms);
/* Flat export (all int64):
 *   ops        [NOPS][8]        rank, round, dst_buf, dst_off, count, acc, src_begin, nsrc
 *   srcs       [NSRCS][3]       peer, buf, off
 *   waits      [NWAITS][4]      rank, round, peer, need_round
 *   exit_waits [NEXIT_WAITS][3] rank, peer, need_round
 *   signals    [NSIGNALS][3]    rank, round, peer
 * buffers ids: 0 = caller input, 1 = caller output, 2 = symmetric scratch.
 * Any pointer may be NULL to skip that table. */
int chb_program_export(const chb_program_t* p, int64_t* ops, int64_t* srcs, int64_t* waits,
                       int64_t* exit_waits, int64_t* signals);
/* names accepted as `algo` for a collective, comma separated */
int chb_list_algorithms(const char* coll, char* out, int outlen);

/* -------------------------------------------------------------- communicators
 * A communicator is driven from one host thread and one stream at a time (like an
 * MPI communicator inside one collective): launches of the same communicator that
 * could overlap on the GPU are not supported.  Every rank must issue the same
 * sequence of collectives.  The first launch of a program uploads its schedule
 * (an allocation and a copy): do it once outside of any stream capture. */
struct chb_comm;
typedef struct CUstream_st* chb_stream_t;   /* cudaStream_t */

size_t chb_heap_bytes(int P, size_t ll_payload_bytes, size_t scratch_bytes, size_t user_bytes);
/* heap_ptrs: P peer-mapped bases of equally laid out, zero-filled heaps (P slices of one
 * local allocation when nlocal == P, the emulated world); mc_ptr: NVLS multicast alias or NULL */
struct chb_comm* chb_comm_create(int rank, int P, int nlocal, void* const* heap_ptrs, void* mc_ptr,
                                 size_t ll_payload_bytes, size_t scratch_bytes, size_t user_bytes,
                                 char* err, int errlen);
/* Native constructors that own their heaps (see boot/bootstrap.h for the rendezvous):
 * all P ranks on the current GPU in this process / one rank per process and GPU of one box. */
struct chb_bootstrap;
struct chb_comm* chb_comm_create_emulated(int P, size_t ll_payload_bytes, size_t scratch_bytes, size_t user_bytes,
                                          char* err, int errlen);
struct chb_comm* chb_comm_create_ipc(struct chb_bootstrap* boot, size_t ll_payload_bytes, size_t scratch_bytes,
                                     size_t user_bytes, char* err, int errlen);
/* the same with heaps from CUDA's virtual-memory allocator and, if want_multicast and every device supports it, an
 * NVLink multicast alias (the multimem kernels then work without Python); *code = CHB_ERR_UNSUPPORTED when the
 * platform has no shareable allocation handles: fall back to chb_comm_create_ipc.  Destroying such a communicator
 * is collective (the ranks meet before memory is unbound and unmapped). */
struct chb_comm* chb_comm_create_vmm(struct chb_bootstrap* boot, size_t ll_payload_bytes, size_t scratch_bytes,
                                     size_t user_bytes, int want_multicast, int* code, char* err, int errlen);
void chb_comm_destroy(struct chb_comm* c);
const char* chb_comm_last_error(const struct chb_comm* c);
int chb_comm_set_timeout_us(struct chb_comm* c, unsigned long long us);
int chb_comm_info(const struct chb_comm* c, int64_t* info, int n);
void* chb_comm_user_ptr(const struct chb_comm* c, int local_index);    /* peer-visible region for caller buffers */
void* chb_comm_scratch_ptr(const struct chb_comm* c, int local_index);
int chb_barrier(struct chb_comm* c, unsigned long long timeout_us, chb_stream_t stream);
/* synchronises the stream; status8 = code, rank, round, peer, expected, seen, launches, epoch */
int chb_comm_status(struct chb_comm* c, int local_index, unsigned long long* status8, chb_stream_t stream);
int chb_comm_clear_error(struct chb_comm* c, chb_stream_t stream);
int chb_comm_trace_enable(struct chb_comm* c, int rounds);
int chb_comm_trace_read(struct chb_comm* c, int local_index, unsigned long long* out, int rounds, chb_stream_t stream);
/* cudaIpc helpers for the one-rank-per-process case */
int chb_ipc_alloc(size_t bytes, void** ptr, void* handle64);
int chb_ipc_open(const void* handle64, void** ptr);
int chb_ipc_close(void* ptr);

/* --------------------------------------------------------------- collectives
 * in / out: one device pointer per local rank.  See chb_compat.h for chb_collective
 * (any algorithm by name) and the reference-compatible entry points. */
int chb_run_program(struct chb_comm* c, const chb_program_t* p, int dtype, int op, const void* const* in,
                    void* const* out, float scale, int nctas, chb_stream_t stream);
/* mode 0 allreduce, 1 reduce-scatter, 2 allgather, 3 two-shot allreduce (flagged lines, no barrier) */
int chb_ll_collective(struct chb_comm* c, int mode, int dtype, int op, const void* const* in, void* const* out,
                      long long count, float scale, int nctas, chb_stream_t stream);
/* mode 0 two-shot allreduce, 1 reduce-scatter, 2 allgather, 3 one-shot allreduce (multimem, sums) */
int chb_nvls_collective(struct chb_comm* c, int mode, int dtype, const void* in, void* out, long long count,
                        float scale, int nctas, chb_stream_t stream);
/* allgather through the bulk-copy (TMA) engine; symmetric input, 16-byte alignment, nbytes % 16 == 0 */
int chb_ag_bulk(struct chb_comm* c, const void* const* in, void* const* out, long long nbytes, int nctas,
                chb_stream_t stream);
int chb_rs_fp8_wire(struct chb_comm* c, int dtype, const void* const* in, void* const* out, long long n,
                    float out_scale, int nctas, chb_stream_t stream);
int chb_rs_adam(struct chb_comm* c, const void* const* grad, void* const* master, void* const* m, void* const* v,
                void* const* param_shard, long long n, const float* hyper, int use_multimem, int nctas,
                chb_stream_t stream);
int chb_adam_flat(const void* grad, void* master, void* m, void* v, void* param_bf16, long long n,
                  const float* hyper, chb_stream_t stream);

int chb_dtype_size(int dtype);
const char* chb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* CHB_H_ */
