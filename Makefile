# Build / test / benchmark entry points (counterpart of the reference's testing/Makefile:
# run-benchmark with RANKS_PER_NODE / NUM_NODES / N_ITER / OVERWRITE, and debug-<impl>).
PKG      := configurable_hierarchical_allreduce_algorithms_b200
PYTHON   ?= python
NGPUS    ?= 8
N_ITER   ?= 12
B        ?= $(NGPUS)
BASE     ?= 1
COLL     ?= allreduce
DTYPE    ?= int32
OVERWRITE ?= 1
RADIX_INCREMENT ?= 1
PORT     ?= 29555
TORCHRUN := $(PYTHON) -m torch.distributed.run --nnodes=1 --nproc-per-node $(NGPUS) --master-addr 127.0.0.1 --master-port $(PORT)

.PHONY: build test test-gpu run-benchmark run-benchmark-native run-benchmark-cpu tune bench clean

build:                 ## compile libchb.so for sm_100a
	$(PYTHON) -m $(PKG)._build -v

test:                  ## CPU tests (schedules, gloo executor, drivers)
	$(PYTHON) -m pytest tests -x -q -m "not gpu"

test-gpu:              ## GPU tests (run on a B200)
	$(PYTHON) -m pytest tests -x -q -m gpu

run-benchmark:         ## sweep of one collective on NGPUS GPUs, CSV like the reference's drivers
	$(TORCHRUN) -m $(PKG).bench.driver $(N_ITER) $(if $(filter 1,$(OVERWRITE)),--overwrite,) b=$(B) base=$(BASE) \
	    coll=$(COLL) dtype=$(DTYPE) radix_increment=$(RADIX_INCREMENT) num_nodes=1

run-benchmark-native:  ## the same sweep by the native launcher (no Python, no MPI: forks one process per GPU)
	$(PKG)/bin/chb_bench $(N_ITER) $(if $(filter 1,$(OVERWRITE)),--overwrite,) ngpus=$(NGPUS) b=$(B) base=$(BASE) \
	    coll=$(COLL) dtype=$(DTYPE) radix_increment=$(RADIX_INCREMENT) num_nodes=1

run-benchmark-cpu:     ## the same sweep over gloo on the host (oversubscribed ranks, like SYSTEM_ENVIRONMENT=LOCAL)
	$(TORCHRUN) -m $(PKG).bench.driver $(N_ITER) $(if $(filter 1,$(OVERWRITE)),--overwrite,) b=$(B) base=$(BASE) \
	    coll=$(COLL) dtype=$(DTYPE) radix_increment=$(RADIX_INCREMENT) backend=gloo reps=5

tune:                  ## measured (algorithm, k, b) table for NGPUS GPUs
	$(TORCHRUN) -m $(PKG).bench.tune

bench:
	$(TORCHRUN) bench.py --gpus $(NGPUS)

debug-%:               ## make debug-allreduce.radix_batch P=8 B=2 : self-checking simulator run of one algorithm
	$(PYTHON) -m $(PKG).bench.debug $(word 1,$(subst ., ,$*)) $(word 2,$(subst ., ,$*)) P=$(NGPUS) b=$(if $(filter $(NGPUS),$(B)),1,$(B))

clean:
	rm -rf $(PKG)/build $(PKG)/bin $(PKG)/libchb.so
