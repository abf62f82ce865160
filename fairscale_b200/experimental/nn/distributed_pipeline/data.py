"""Edge record of the module graph (parity: fairscale/experimental/nn/distributed_pipeline/data.py:10-18)."""

from dataclasses import dataclass
from typing import Generic, TypeVar

ConsumerType = TypeVar("ConsumerType")


@dataclass
class DataConsumer(Generic[ConsumerType]):
    """``consumer`` takes, as its input number ``consumer_input_idx``, output number ``output_idx`` of the producer."""

    consumer: ConsumerType
    consumer_input_idx: int
    output_idx: int
