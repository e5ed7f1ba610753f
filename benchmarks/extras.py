"""Extra records that bench.py appends to its JSON line (see `run`)."""


def run(ctx, kv, args, elapsed_s):
    return {}
