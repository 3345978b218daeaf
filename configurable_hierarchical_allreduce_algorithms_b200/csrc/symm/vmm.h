/* Native symmetric heap over CUDA virtual-memory allocations, with an optional NVLink multicast alias
 * (see vmm.cc).  Collective over the ranks of a bootstrap; one heap per rank on its current device. */
#ifndef CHB_VMM_H_
#define CHB_VMM_H_
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

struct chb_bootstrap;
typedef struct chb_vmm_heap chb_vmm_heap;

/* want_multicast != 0: also create the multicast alias when every rank's device supports it.
 * CHB_ERR_UNSUPPORTED (on every rank alike) when the driver or shareable handles are missing. */
int chb_vmm_create(struct chb_bootstrap* boot, size_t bytes, int want_multicast, chb_vmm_heap** out, char* err, int errlen);
/* collective as well: the ranks meet before anything is unmapped, and again before anything is released */
void chb_vmm_destroy(chb_vmm_heap* h);
void* chb_vmm_ptr(const chb_vmm_heap* h, int rank);        /* rank's heap as mapped here */
void* chb_vmm_multicast_ptr(const chb_vmm_heap* h);        /* alias of all heaps, or NULL */
size_t chb_vmm_bytes(const chb_vmm_heap* h);               /* mapped size (the request rounded up) */
/* the rounding rule, exposed for tests */
size_t chb_vmm_mapped_size(size_t bytes, size_t mem_granularity, size_t mc_granularity);

#ifdef __cplusplus
}
#endif
#endif
