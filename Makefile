# Wrappers in the manner of the reference's Makefile (targets that wrap cargo and scripts there).
PY ?= python

.PHONY: build test test-gpu replay bench

build:            ## compile the CUDA kernels for sm_100a (in-tree, csrc/_build)
	$(PY) -c "import __graft_entry__ as g; g.build()"

test:             ## what runs without a GPU
	$(PY) -m pytest tests -x -q -m "not gpu"

test-gpu:         ## on a B200
	$(PY) -m pytest tests -x -q -m gpu

replay:           ## usage of the trace replay program
	bin/trace_run --help

bench:            ## one JSON line: decode tokens/s at the 0.6B shape, batch 8, context 4096
	$(PY) bench.py
