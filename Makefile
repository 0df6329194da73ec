# Developer commands (the counterparts of the reference's justfile).
.PHONY: build format-check format-fix lint-check lint-fix type-check spell-check check fix test test-gpu

build:
	python -c "from yafsdp_b200 import _native; print(_native.build())"

format-check:
	ruff format --check

format-fix:
	ruff format

lint-check:
	ruff check

lint-fix:
	ruff check --fix

type-check:
	mypy

spell-check:
	codespell

check: format-check lint-check type-check spell-check

fix: format-fix lint-fix

test:
	python -m pytest tests -q -m "not gpu"

test-gpu:
	python -m pytest tests -q -m gpu
