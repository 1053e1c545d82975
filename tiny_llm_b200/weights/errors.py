class WeightError(ValueError):
    """The weights do not fit the model: the message lists every missing tensor, every unexpected
    tensor and every tensor of the wrong shape or kind at once."""
