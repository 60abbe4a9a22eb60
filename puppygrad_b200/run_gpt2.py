"""`run-gpt2` of the reference's command line (puppygrad src/main.rs:1305-1388) on this backend:

    python -m puppygrad_b200.run_gpt2 --model-dir DIR --prompt "..." [--stats] [--stream-raw-tokens]
"""
import sys

from .runtime import run_gpt2

if __name__ == "__main__":
    sys.exit(run_gpt2())
