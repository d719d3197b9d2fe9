import contextlib


class MemSnapshotsProfiler:
    def __init__(self, *a, **k):
        pass


class PyTorchProfiler:
    def __init__(self, *a, **k):
        pass


@contextlib.contextmanager
def profile(*a, **k):
    yield None


def step():
    pass
