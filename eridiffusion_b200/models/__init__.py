from .registry import build_model, known_models, register_model  # noqa: F401
from . import mmdit  # noqa: F401  (registers "flux", "tiny_mmdit")
from . import ltx_video  # noqa: F401  (registers "ltx_video")
