"""Context-parallel hooks of the BSA path: ``context_parallel_util`` (process state) and
``ulysses_wrapper`` (the all-to-all pair and its decorator), importable by the same module names as
in the reference (``from ...context_parallel.ulysses_wrapper import ulysses_wrapper``)."""
