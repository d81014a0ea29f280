from .req import FinishStatus, Req, TokenHealingReq  # noqa: F401
from .sampling_params import ParamError, SamplingParams  # noqa: F401
from .start_args import StartArgs, get_env_start_args, set_env_start_args  # noqa: F401
