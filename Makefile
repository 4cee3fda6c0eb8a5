# Convenience targets. The kernel library is built in-tree; nothing is installed system-wide.
.PHONY: build test gputest lint clean

build:
	python -m msamp.ops.build

test: build
	python -m pytest tests -q -m "not gpu"

gputest: build
	python -m pytest tests -q -m gpu

lint:
	python -m flake8 --max-line-length 140 msamp tests bench.py

clean:
	rm -rf msamp/ops/build msamp/ops/libmsamp_b200.so
