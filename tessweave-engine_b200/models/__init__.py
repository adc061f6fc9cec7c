"""Models: a generic assembly of parts, and the architectures described with it."""
from .spec import LayerSpec, ModelSpec, ScheduleEntry
from .model import Model
from . import qwen2  # noqa: F401  (registers "Qwen2ForCausalLM")
from . import linurax  # noqa: F401  (registers "Linurax")
from . import sapatar  # noqa: F401  (registers "Sapatar")
from . import nufatar  # noqa: F401  (registers "Nufatar")
from . import dugudra  # noqa: F401  (registers "Dugudra")

__all__ = ["LayerSpec", "ModelSpec", "ScheduleEntry", "Model"]
