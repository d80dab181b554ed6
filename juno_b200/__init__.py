"""juno_b200 — B200 (sm_100a) decode backend behind Juno's MatVec / ForwardPassHandler / InferencePipeline API."""
from . import synth  # noqa: F401
from ._lib import JunoError  # noqa: F401
