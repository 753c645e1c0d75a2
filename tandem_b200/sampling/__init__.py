from tandem_b200.sampling.params import SamplingParams

__all__ = ["SamplingParams"]
