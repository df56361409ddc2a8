class WeightsError(RuntimeError):
    """A weights file that cannot be read, or whose tensors do not fit the model."""
