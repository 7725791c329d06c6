from .datacollectors import GeneratorWeightWorker, SyncLLMCollector, VLLMWorkerWrapper
from .metric_logger import MetricLoggerWorker
from .parameter_servers import BroadcastParameterServer, ParameterServer, VLLMParameterServer
from .postprocessing import PostProcessingWorker
from .replay import ReplayBuffer
from .trainers import TrainingWorker
from .weight_updaters import WeightUpdateReceiver

# names of the reference's engine-specific classes (torchtune/dev/rl/workers/__init__.py:7-21); the roles are the same
VLLMHFWeightUpdateReceiver = WeightUpdateReceiver

__all__ = ["SyncLLMCollector", "MetricLoggerWorker", "ParameterServer", "PostProcessingWorker", "ReplayBuffer", "TrainingWorker", "WeightUpdateReceiver",
           "VLLMParameterServer", "VLLMHFWeightUpdateReceiver", "BroadcastParameterServer", "GeneratorWeightWorker", "VLLMWorkerWrapper"]
