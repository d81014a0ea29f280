"""Imports every model module so their @register_model decorators run."""
from . import llama  # noqa: F401
from . import qwen3_moe  # noqa: F401
from . import deepseek2  # noqa: F401
from . import generic  # noqa: F401
from . import qwen2_vl  # noqa: F401
from . import gpt_oss  # noqa: F401
from . import llava  # noqa: F401
from . import internvl  # noqa: F401
from . import qwen3_next  # noqa: F401
from . import qwen3_omni  # noqa: F401
from . import deepseek_v32  # noqa: F401
from . import gemma4  # noqa: F401
