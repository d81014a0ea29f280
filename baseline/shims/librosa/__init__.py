"""Import-time stand-in for `librosa` (audio decoding is not used by the text benchmark)."""


def load(*a, **k):
    raise RuntimeError("librosa is not available in this environment")
