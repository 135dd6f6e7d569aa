"""Error types (crates/core/src/error.rs:8-46)."""


class CoreError(Exception):
    """Base class of framework errors."""


class ShapeMismatch(CoreError):
    def __init__(self, expected, actual, what: str = ""):
        super().__init__(f"shape mismatch{(' in ' + what) if what else ''}: expected {tuple(expected)}, got {tuple(actual)}")
        self.expected, self.actual = tuple(expected), tuple(actual)


class InvalidShape(CoreError):
    pass


class InvalidArgument(CoreError):
    pass


class BackendError(CoreError):
    pass


class SerializationError(CoreError):
    pass
