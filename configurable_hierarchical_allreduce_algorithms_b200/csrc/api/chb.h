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

int chb_dtype_size(int dtype);
const char* chb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* CHB_H_ */
