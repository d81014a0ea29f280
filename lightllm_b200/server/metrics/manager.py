"""Metric manager process: owns the Prometheus registry so that several HTTP workers and the router
report into one place.  Clients send fire-and-forget updates over a zmq PUSH socket and fetch the
exposition text with a REQ/REP call; an optional thread pushes to a gateway.
Reference: lightllm/server/metrics/manager.py (rpyc service + push-gateway thread).
"""
from __future__ import annotations

import threading
import time
import traceback

import zmq

from ..core.objs.start_args import StartArgs, set_env_start_args
from .metrics import Monitor


def _addr(args, suffix):
    from ..router.manager import zmq_addr

    return zmq_addr(args, f"{args.metric_port}_{suffix}")


def gateway_auth_handler(url, method, timeout, headers, data):
    """`--enable_monitor_auth`: pushes to the gateway carry HTTP basic auth taken from the environment
    (reference: lightllm/server/metrics/metrics.py:38-43)."""
    import os

    from prometheus_client.exposition import basic_auth_handler

    user, password = os.getenv("USERNAME"), os.getenv("PASSWORD")
    if user is None or password is None:
        raise ValueError("--enable_monitor_auth needs the USERNAME and PASSWORD environment variables")
    return basic_auth_handler(url, method, timeout, headers, data, user, password)


class MetricServer:
    def __init__(self, args: StartArgs):
        self.args = args
        self.monitor = Monitor(args.model_name)
        ctx = zmq.Context(1)
        self.pull = ctx.socket(zmq.PULL)
        self.pull.bind(_addr(args, "push"))
        self.rep = ctx.socket(zmq.REP)
        self.rep.bind(_addr(args, "req"))
        self.poller = zmq.Poller()
        self.poller.register(self.pull, zmq.POLLIN)
        self.poller.register(self.rep, zmq.POLLIN)
        if args.metric_gateway:
            threading.Thread(target=self._push_loop, daemon=True).start()

    def _push_loop(self):
        from prometheus_client import push_to_gateway

        grouping = dict(kv.split("=", 1) for kv in (self.args.grouping_key or []) if "=" in kv)
        kw = {}
        if getattr(self.args, "enable_monitor_auth", False):     # basic auth from the USERNAME / PASSWORD variables
            kw["handler"] = gateway_auth_handler
        while True:
            time.sleep(self.args.push_interval)
            try:
                push_to_gateway(self.args.metric_gateway, job=self.args.job_name, registry=self.monitor.registry,
                                grouping_key=grouping, **kw)
            except Exception:
                pass

    def serve(self):
        while True:
            for sock, _ in self.poller.poll(1000):
                if sock is self.pull:
                    kind, name, value = self.pull.recv_pyobj()
                    getattr(self.monitor, kind)(name, value)
                else:
                    self.rep.recv()
                    self.rep.send(self.monitor.generate_latest())


class MetricClient:
    """Used by HTTP workers and the router; never blocks the caller."""

    def __init__(self, args: StartArgs):
        ctx = zmq.Context.instance()
        self.push = ctx.socket(zmq.PUSH)
        self.push.setsockopt(zmq.SNDHWM, 10000)
        self.push.connect(_addr(args, "push"))
        self.req_addr = _addr(args, "req")
        self._ctx = ctx

    def _send(self, kind, name, value):
        try:
            self.push.send_pyobj((kind, name, value), zmq.NOBLOCK)
        except zmq.ZMQError:
            pass

    def counter_inc(self, name, v=1.0):
        self._send("counter_inc", name, v)

    def gauge_set(self, name, v):
        self._send("gauge_set", name, v)

    def histogram_observe(self, name, v):
        self._send("histogram_observe", name, v)

    def generate_latest(self, timeout_ms: int = 2000) -> bytes:
        s = self._ctx.socket(zmq.REQ)
        s.setsockopt(zmq.LINGER, 0)
        s.connect(self.req_addr)
        try:
            s.send(b"get")
            if s.poll(timeout_ms):
                return s.recv()
            return b""
        finally:
            s.close()


def start_metric_manager(args_dict: dict, pipe_writer):
    from ...utils.process_utils import graceful_registry, set_proc_title, start_parent_check_thread

    args = StartArgs.from_dict(args_dict)
    set_env_start_args(args)
    set_proc_title(f"lightllm::{args.unique_server_name}::metric_manager")
    graceful_registry("metric")
    start_parent_check_thread()
    try:
        srv = MetricServer(args)
    except Exception:
        pipe_writer.send(traceback.format_exc())
        raise
    pipe_writer.send("init ok")
    srv.serve()
