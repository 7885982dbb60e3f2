# Developer entry points.  `make build` needs nvcc (cross-compiles sm_100a without a GPU) and g++.
PY ?= python

.PHONY: build test test-gpu sanitize bench clean

build:
	$(PY) -m recsdk_b200._build

test: build
	$(PY) -m pytest tests -q -m "not gpu"

test-gpu: build
	$(PY) -m pytest tests -q -m gpu

# host engines under ThreadSanitizer and ASan + UBSan (csrc/host/stress/host_stress.cpp)
sanitize:
	$(PY) -m pytest tests/test_host_sanitizers.py -q

bench: build
	$(PY) bench.py

clean:
	rm -rf build recsdk_b200/_C_cuda.so recsdk_b200/_C_host*.so
