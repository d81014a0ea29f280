"""Entry point:  python -m lightllm_b200.server.api_server --model_dir <hf dir> --tp 8 ...
(reference: lightllm/server/api_server.py)."""
from __future__ import annotations

import multiprocessing as mp

from .api_cli import make_argument_parser
from .core.objs.start_args import StartArgs


def launch_server(args: StartArgs):
    from .api_start import config_server_start, normal_or_p_d_start, pd_master_start, visual_only_start

    try:
        mp.set_start_method("spawn")
    except RuntimeError:
        pass
    if args.run_mode == "pd_master":
        pd_master_start(args)
    elif args.run_mode == "config_server":
        config_server_start(args)
    elif args.run_mode == "visual_only":
        visual_only_start(args)
    else:
        normal_or_p_d_start(args)


if __name__ == "__main__":
    launch_server(StartArgs.from_namespace(make_argument_parser().parse_args()))
