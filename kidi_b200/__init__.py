"""kidi_b200: a small model library with generation of its own, for one B200.

From a model folder (config.json, model.safetensors) or from a configuration and a
seed to generated tokens: typed configuration and registry, weights by name, layers
put together from parts, a paged cache with a slot per sequence, one step function,
a generation loop with greedy and temperature sampling, and hand-written CUDA kernels
for sm_100a underneath.

The Python entry point follows the reference's (`kidi.main(args) -> int`,
python/kidi/__init__.py:11-13): `kidi_b200.main(["generate", "-m", DIR, ...])` runs the
command line and returns its exit code.
"""
from .errors import ErrorCode, KidiError
from .engine.plan import StepBatch
from .engine.engine import Engine
from .registry import register_architecture, registered_architectures
from .parts.registry import register_part
from .weights.random_init import write_random_model

__version__ = "0.1.0"


def main(args=None) -> int:
    from .cli import main as cli_main
    return cli_main(args)


__all__ = ["Engine", "ErrorCode", "KidiError", "StepBatch", "main", "register_architecture", "register_part",
           "registered_architectures", "write_random_model", "__version__"]
