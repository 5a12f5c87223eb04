# Convenience targets; everything they do is a plain command of the package (see README.md).
PY ?= python

.PHONY: build test test-gpu docs bench clean

build:            ## compile the native code for sm_100a (no GPU needed)
	$(PY) -m rocm_systems_b200.utils.build

test: build       ## CPU tier
	$(PY) -m pytest tests -q -m "not gpu"

test-gpu: build   ## GPU tier (on a B200 box)
	$(PY) -m pytest tests -q -m gpu

docs:             ## regenerate the references that are generated from the code
	$(PY) -m rocm_systems_b200.utils.apidoc > docs/python_api.md
	$(PY) -m rocm_systems_b200.utils.apidoc --c > docs/c_api.md

bench:            ## the headline training step on one GPU
	$(PY) bench.py --steps 5 --warmup 3

clean:            ## built objects and libraries (sources stay)
	rm -rf rocm_systems_b200/build rocm_systems_b200/lib rocm_systems_b200/bin
