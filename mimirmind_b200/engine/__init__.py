"""Engine: model assembly, cache storage, the step function, scheduler and generation."""
