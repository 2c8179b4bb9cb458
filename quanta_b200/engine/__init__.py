"""Model, step function, scheduler and generation."""
