"""Import-only stand-in for `ray`, so that the reference's placement and
simulator modules can be imported for differential tests.  Nothing here runs
remotely: `remote` hands the function back and `get`/`put` are identities."""
from . import actor, util  # noqa: F401


def remote(*args, **kwargs):
    if len(args) == 1 and callable(args[0]) and not kwargs:
        return args[0]

    def wrap(fn):
        return fn
    return wrap


def is_initialized():
    return False


def init(*args, **kwargs):
    return None


def get(x):
    return x


def put(x):
    return x
