"""Status codes and the exception shared by the C-ABI bindings."""
SMOL_OK = 0
SMOL_ERR_INVALID = -1
SMOL_ERR_UNBOUND = -2
SMOL_ERR_CUDA = -3
SMOL_ERR_UNSUPPORTED = -4
SMOL_ERR_CAPACITY = -5


class SmolError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"smoltts_b200 error {code}: {message}")
        self.code = code
