"""Configuration errors.

The classes mirror the three failure kinds of the reference's config parser
(crates/arch/src/llama.rs:305-317 unknown architecture, :319-325 missing key,
:332-370 invalid value) so that callers can tell them apart.
"""


class ConfigError(ValueError):
    """Base class of every configuration failure."""


class MissingKey(ConfigError):
    def __init__(self, key: str):
        super().__init__(f"config.json: required key '{key}' is missing")
        self.key = key


class InvalidValue(ConfigError):
    def __init__(self, key: str, why: str):
        super().__init__(f"config.json: invalid value for '{key}': {why}")
        self.key = key
        self.why = why


class UnknownArchitecture(ConfigError):
    def __init__(self, name: str, supported):
        super().__init__(
            f"config.json: architecture '{name}' is not registered; "
            f"registered architectures: {sorted(supported)}")
        self.name = name
