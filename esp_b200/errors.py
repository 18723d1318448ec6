"""Error classes of the library, named after the reference's ``InferError``
variants (crates/esp/src/infer/provider.rs:160-183)."""


class InferError(Exception):
    """Base class of every error the library raises on purpose."""


class InvalidConfig(InferError):
    """config.json holds a value that cannot describe a model."""


class Unsupported(InferError):
    """A named feature of config.json (or of a request) is not implemented."""

    def __init__(self, feature: str, detail: str):
        super().__init__(f"unsupported {feature}: {detail}")
        self.feature = feature
        self.detail = detail


class InvalidWeights(InferError):
    """The checkpoint does not match what the configuration calls for."""


class InvalidRequest(InferError):
    """A request or a step asks for something that cannot be run."""


class PromptTooLong(InferError):
    def __init__(self, length: int, limit: int):
        super().__init__(f"prompt of {length} tokens does not fit the context window of {limit}")
        self.length = length
        self.limit = limit


class CacheFull(InferError):
    """The cache has no free slot or page left for the step."""


class Backend(InferError):
    """The device or the compiled kernels failed or are missing."""


class NonFiniteScores(Backend):
    """A step's logits held a NaN or an infinity: no token may be decided from them."""
