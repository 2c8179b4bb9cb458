"""Sampling options and the device sampler."""
