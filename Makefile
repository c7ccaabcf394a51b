# Convenience targets; everything they run is documented in docs/development.md.
PY ?= python

.PHONY: build test test-gpu bench bench-cpu clean

build:            ## nvcc (sm_100a) + g++: ops, storage engine, token index (in-tree shared objects)
	$(PY) -m daser_b200.ops.build

test: build       ## CPU suite (control plane, IO engine, native index, services, gloo ranks, sanitizers)
	$(PY) -m pytest tests -q -m "not gpu"

test-gpu: build   ## on a B200
	$(PY) -m pytest tests -q -m gpu

bench: build      ## headline benchmark on one GPU
	$(PY) bench.py

bench-cpu: build  ## benchmarks that need no GPU
	cd benchmarks && $(PY) bench_control_plane.py && $(PY) bench_storage.py --device cpu && $(PY) bench_frontend.py

clean:
	rm -rf build daser_b200/ops/libdaser_ops.so daser_b200/io/libdaser_io.so daser_b200/server/libdaser_index.so
