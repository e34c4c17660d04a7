"""CPU oracle for the Universal-LM-Trainer training hot path.

TEST INFRASTRUCTURE ONLY.  Nothing that ships (the ``universal-lm-trainer_b200``
package, its CUDA library) may import this package: it exists so that the test
suite, the smoke check and the CPU-baseline leg of the benchmark can compare the
CUDA kernels against a plain restatement of the reference's PyTorch path.

Every function names the reference lines it restates (paths are relative to the
root of sunyi9161/Universal-LM-Trainer).  The restatement is pinned against
vectors produced by importing the reference itself (``tests/golden``): the
reference ships no golden vectors or known-answer tests of its own for this
path, so those fixtures are the pin.
"""
from . import ops, batching, model, infer  # noqa: F401
