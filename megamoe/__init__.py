"""Drop-in import name: `import megamoe` resolves to the B200 implementation in deepgemm_b200.megamoe."""
from deepgemm_b200.megamoe import *  # noqa: F401,F403
from deepgemm_b200.megamoe import (  # noqa: F401
    __all__, __version__, _large_opt_3stage_mode, _large_opt_3stage_selected, _large_opt_3stage_threshold,
    _staged_as_split_launches,
)
