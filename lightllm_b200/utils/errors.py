"""Error types mapped to HTTP status codes by the API layer (reference: lightllm/utils/error_utils.py,
lightllm/server/api_errors.py)."""


class ServerBusyError(Exception):
    """Admission refused (HTTP 429)."""

    def __init__(self, message="Server is busy, please try again later.", status_code=429):
        super().__init__(message)
        self.message = message
        self.status_code = status_code


class NixlPrefillNodeStopGenToken(Exception):
    pass


class CommTimeout(RuntimeError):
    """A bounded device-side wait on a peer ran out; the step's result is invalid."""
