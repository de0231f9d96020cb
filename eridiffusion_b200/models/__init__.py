from .registry import build_model, known_models, register_model  # noqa: F401
from . import mmdit  # noqa: F401  (registers "flux", "tiny_mmdit")
from . import ltx_video  # noqa: F401  (registers "ltx_video")
from . import sdxl_unet  # noqa: F401  (registers "sdxl")
from . import nextdit  # noqa: F401  (registers "zimage", "wan22")
from . import sd35_klein  # noqa: F401  (registers "sd35", "klein")
from . import text_encoders  # noqa: F401  (registers "clip_l", "open_clip_g", "t5_encoder", "qwen3_encoder", "gemma3_encoder")
from . import vae  # noqa: F401  (registers "vae_sdxl", "vae_flux")
from . import families  # noqa: F401  (registers "krea", "hunyuan", "hidream", "lumina", "omnigen2", "qwen_edit_image")
