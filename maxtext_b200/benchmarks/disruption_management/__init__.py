"""Disruption harness: run a training job, disturb it on purpose (pre-emption notice or a killed rank), restart it the way a
cluster scheduler would, and measure what the disruption cost (benchmarks/disruption_management/ in the reference, which
drives pods through kubectl; here the job is a set of local rank processes)."""
from .disruption_manager import Disruption, DisruptionManager, StepMonitor          # noqa: F401
