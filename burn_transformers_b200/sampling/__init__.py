from .config import GenerationConfig
from .random import interior_unit_f32, sequence_stream, splitmix64, uniform
from .tracker import FinishReason, GeneratedSequence, SequenceTracker, longest_stop_suffix, stop_decision

__all__ = ["GenerationConfig", "interior_unit_f32", "sequence_stream", "splitmix64", "uniform", "FinishReason",
           "GeneratedSequence", "SequenceTracker", "longest_stop_suffix", "stop_decision"]
