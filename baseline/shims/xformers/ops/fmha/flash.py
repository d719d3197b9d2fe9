class FwOp:
    OPERATOR = None
