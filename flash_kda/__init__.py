"""Drop-in module name of the reference (`import flash_kda`): flash-linear-attention's
`chunk_kda` backend dispatch looks for a top-level module of this name exposing `fwd`
(reference: flash_kda/__init__.py:2-5).  The implementation lives in `flashkda_b200`."""
from flashkda_b200 import fwd, get_workspace_size

__all__ = ["fwd", "get_workspace_size"]
