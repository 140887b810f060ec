"""Sampling options, the host twin and the device kernels' face."""

from .sampler import (SamplingParams, device_choose, host_argmax, host_sample, host_survivors, uniform_for)

__all__ = ["SamplingParams", "device_choose", "host_argmax", "host_sample", "host_survivors", "uniform_for"]
