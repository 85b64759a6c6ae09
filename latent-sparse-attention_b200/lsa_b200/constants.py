"""Values callers and kernels have to agree on (the reference keeps them in src/lsa/constants.py)."""


class Sentinel:
    # The only padding value an id list carries
    PAD: int = -1


class Math:
    NINF: float = float("-inf")
    # Norm floor of a row normalisation: a zero row stays zero
    NORM_EPS: float = 1e-12


class Rotary:
    NONE: str = "none"
    PREFIX: str = "prefix"
    SUFFIX: str = "suffix"
    ENDS: tuple = (NONE, PREFIX, SUFFIX)


class Chunk:
    # Query rows a sparse read takes at a time
    QUERY: int = 512


class PackedKey:
    # The key of no bucket: the least int64
    EMPTY: int = -(2**63)
