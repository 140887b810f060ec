"""Error types of the library.

Errors are values with a kind, in the manner of the reference's `HerbertError`
(crates/core/src/error.rs:9-30: Io / ModelLoad / Tensor / Config / Backend /
Serialization / SafeTensors).  Every public call validates its inputs on the host
and raises one of these before anything is launched on the device.
"""


class HerbertError(Exception):
    """Base class of every error the library raises on purpose."""


class ConfigError(HerbertError):
    """config.json is missing a key, holds an invalid value, or asks for something unsupported."""


class WeightError(HerbertError):
    """A model folder's tensors do not match what the model needs."""


class SafeTensorsError(WeightError):
    """The container file itself is malformed (truncated, bad header, unknown dtype)."""


class CacheError(HerbertError):
    """A cache request cannot be served: no free slot or page, bad slot, double free."""


class BackendError(HerbertError):
    """The device path is unavailable or refused an input (missing extension, unsupported size)."""


class RequestError(HerbertError):
    """A step or generation request is malformed (empty, token id out of range, too long)."""
