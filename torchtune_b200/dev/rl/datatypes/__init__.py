from .request_output import CompletionOutput, RequestOutput
from .trajectory import Trajectory

# the reference names the per-sample record after its inference engine; the fields are the same
VllmCompletionOutput = CompletionOutput

__all__ = ["CompletionOutput", "RequestOutput", "Trajectory", "VllmCompletionOutput"]
