"""Placeholder replaced below."""


def try_run(opt, state, group, grads, params):
    return False
