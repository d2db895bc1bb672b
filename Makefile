# Build, check and measure (the counterpart of the reference's benchmark/docker/build_and_run.sh:
# compile the kernel library, run the backend verification, the tests and the benchmarks).
PY ?= python
NGPU ?= 1

.PHONY: build test test-gpu verify bench benchspec microbench all

all: build verify test

build:            ## compile csrc/*.cu for sm_100a into gonn_b200/_C/libgonn_b200.so
	$(PY) -m gonn_b200.build

test:             ## CPU tests (oracle paths, TCP and gloo ranks)
	$(PY) -m pytest tests -q -m "not gpu"

test-gpu:         ## GPU tests (needs a B200 and the built library)
	$(PY) -m pytest tests -q -m gpu

verify:           ## backend against independent numpy formulas; exits non-zero on a mismatch
	$(PY) -m gonn_b200.utils.verify

bench:            ## flagship training step on NGPU GPUs of this node
ifeq ($(NGPU),1)
	$(PY) bench.py --gpus 1
else
	$(PY) -m torch.distributed.run --nnodes=1 --nproc-per-node $(NGPU) --master-addr 127.0.0.1 bench.py --gpus $(NGPU)
endif

benchspec:        ## the reference's cross-framework benchmark specification + aggregated table
	$(PY) -m gonn_b200.utils.benchspec run --out benchmark/results
	$(PY) -m gonn_b200.utils.benchspec aggregate benchmark/results > benchmark/RESULTS.md

microbench:       ## kernel micro-benchmarks (GEMM, attention, elementwise, norm, reference attention shapes)
	for k in gemm flash elementwise norm refattn; do $(PY) -m gonn_b200.utils.microbench $$k; done
