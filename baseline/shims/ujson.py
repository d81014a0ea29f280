"""Minimal stand-in for `ujson`."""
from json import *  # noqa: F401,F403
from json import dumps, loads  # noqa: F401
