"""Building blocks of the asynchronous GRPO orchestrator: example buffer with difficulty pools, rollout scheduler, rollout filters,
advantage functions and the adaptive rollout-depth controller.

Parity: surogate/grpo/orchestrator/{buffer,scheduler,filters,advantage,depth_controller}.py.
"""
from .advantage import AdvantageInputs, AdvantageOutputs, compute_advantages, default_advantage, std_normalized_advantage  # noqa: F401
from .buffer import BufferConfig, ExampleBuffer  # noqa: F401
from .depth import DepthObservation, RolloutDepthController  # noqa: F401
from .filters import FilterResult, GibberishFilter, RepetitionFilter, apply_filters, make_filters  # noqa: F401
from .scheduler import RolloutScheduler, SchedulerConfig  # noqa: F401
from .loop import AsyncOrchestrator, AsyncOrchestratorConfig, OrchestratorCheckpoints, Progress, async_config_from, make_generate_group  # noqa: F401
from .evaluation import evaluate_policy, pass_at_k  # noqa: F401
