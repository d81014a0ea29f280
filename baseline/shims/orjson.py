"""Minimal stand-in for `orjson` on top of the standard json module."""
import json

OPT_INDENT_2 = 1
OPT_SORT_KEYS = 2
OPT_NON_STR_KEYS = 4
JSONDecodeError = json.JSONDecodeError


def dumps(obj, default=None, option=0):
    return json.dumps(obj, default=default, indent=2 if option & OPT_INDENT_2 else None,
                      sort_keys=bool(option & OPT_SORT_KEYS)).encode()


def loads(s):
    return json.loads(s)
