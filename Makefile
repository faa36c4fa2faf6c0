.PHONY: build test test-fast test-gpu lint clean

build:
	python -m odc_b200.build

test:
	python -m pytest tests -q -m "not gpu"

# the CPU tests four at a time (pytest-xdist); the GPU tests always run one at a time
test-fast:
	python -m pytest tests -q -m "not gpu" -n 4

test-gpu:
	python -m pytest tests -q -m gpu

lint:
	python -m compileall -q odc_b200 examples tests bench.py __graft_entry__.py

clean:
	rm -rf odc_b200/csrc/build odc_b200/_C.so
