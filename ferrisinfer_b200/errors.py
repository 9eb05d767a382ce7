"""Error types of the engine.

The reference keeps one error struct with a kind tag
(crates/ferrisinfer-core/src/error.rs:5-22: Io, Parse, InvalidShape,
InvalidLayout, InvalidType, InvalidConfig, MissingWeight, Unsupported,
Runtime).  Here each kind that a caller may want to catch is an exception
class of its own.
"""

from __future__ import annotations


class FerrisError(Exception):
    """Base class of every error the engine raises on purpose."""


class ConfigError(FerrisError):
    """config.json is missing a key, has a wrong type, or fails validation."""


class UnsupportedError(FerrisError):
    """The model folder asks for something this engine does not run."""


class WeightFileError(FerrisError):
    """A safetensors file is malformed (header, offsets, dtype)."""


class WeightLoadError(FerrisError):
    """The tensors of a model folder do not fit the model.

    One error carries everything that is wrong, so a user fixes the folder in
    one go: ``missing`` (names the model needs), ``unexpected`` (names the model
    does not know) and ``wrong_shape`` ((name, expected, found) triples).
    """

    def __init__(self, missing, unexpected, wrong_shape, where=""):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"weights do not fit the model{(' in ' + where) if where else ''}:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}):")
            lines += [f"    {n}" for n in self.missing]
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}):")
            lines += [f"    {n}" for n in self.unexpected]
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}):")
            lines += [
                f"    {n}: expected {list(e)}, found {list(f)}" for n, e, f in self.wrong_shape
            ]
        super().__init__("\n".join(lines))


class KernelError(FerrisError):
    """A CUDA kernel refused its arguments, or the extension is unavailable."""


class CacheError(FerrisError):
    """The cache manager was asked for something it cannot give."""


class OutOfPages(CacheError):
    """The page pool has fewer free pages than an allocation needs."""


class SchedulerError(FerrisError):
    """A request that the scheduler cannot ever run (too long, empty...)."""
