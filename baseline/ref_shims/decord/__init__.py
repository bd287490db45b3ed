"""Stand-in for ``decord`` (video reader of the reference datasets; unused with synthetic batches)."""


class VideoReader:
    def __init__(self, *args, **kwargs):
        raise RuntimeError("decord is not installed in this image; video samples are unavailable")


def cpu(*args, **kwargs):
    return None
