# Convenience targets; every command is also documented in README.md.
PY ?= python

.PHONY: build test test-gpu bench smoke clean

build:            ## compile the sm_100a kernel library and the native data loader in-tree (no GPU needed)
	$(PY) -m cppmega_b200.ops.cuda.build
	$(PY) -m cppmega_b200.runtime.build

test:             ## CPU suite (gloo for the multi-rank tests)
	$(PY) -m pytest tests -q -m "not gpu"

test-gpu:         ## on a B200 (multi-GPU tests run when more than one GPU is visible)
	$(PY) -m pytest tests -q -m gpu

bench:            ## headline benchmark on one GPU; N GPUs: torch.distributed.run --nproc-per-node N bench.py --gpus N
	$(PY) bench.py --steps 5 --warmup 3

smoke:
	$(PY) -c "import __graft_entry__ as g; g.build(); g.smoke()"

clean:
	rm -rf cppmega_b200/ops/cuda/_build
	rm -f cppmega_b200/ops/cuda/libcppmega_b200_kernels.so
