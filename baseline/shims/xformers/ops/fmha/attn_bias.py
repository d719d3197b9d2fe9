class AttentionBias:
    pass


class _Unavailable(AttentionBias):
    def __init__(self, *a, **k):
        raise NotImplementedError("xformers is not installed")

    @classmethod
    def from_seqlens(cls, *a, **k):
        raise NotImplementedError("xformers is not installed")


class LowerTriangularMask(_Unavailable):
    pass


class LowerTriangularFromBottomRightMask(_Unavailable):
    pass


class LocalAttentionFromBottomRightMask(_Unavailable):
    pass


class BlockDiagonalMask(_Unavailable):
    pass


class BlockDiagonalCausalMask(_Unavailable):
    pass
