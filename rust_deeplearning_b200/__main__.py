"""`python -m rust_deeplearning_b200 MODEL_DIR ...` is the command line of `bin/rustml-infer`."""
import sys

from .cli import main

sys.exit(main())
