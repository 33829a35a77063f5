.PHONY: build test test-gpu bench clean

build:
	python -m popxl_addons_b200.build

test: build
	python -m pytest tests -q -m "not gpu"

test-gpu: build
	python -m pytest tests -q -m gpu

bench: build
	python bench.py

clean:
	rm -rf popxl_addons_b200/lib build *.egg-info
	find . -name __pycache__ -type d -prune -exec rm -rf {} +
