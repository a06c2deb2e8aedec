"""Configuration errors.

The kinds follow the reference's `ConfigError`
(crates/model/src/config/errors.rs:11-35), but here a missing required key is
raised; the reference falls back to silent defaults
(crates/model/src/config/model_config.rs:329-336).
"""


class ConfigError(ValueError):
    """Base of all configuration errors."""


class UnknownArchitecture(ConfigError):
    def __init__(self, name, registered):
        self.name = name
        self.registered = sorted(registered)
        super().__init__(f"unknown architecture: {name!r}; registered: {', '.join(self.registered) or '(none)'}")


class MissingField(ConfigError):
    def __init__(self, field):
        self.field = field
        super().__init__(f"missing required field: {field}")


class InvalidField(ConfigError):
    def __init__(self, field, message):
        self.field = field
        self.message = message
        super().__init__(f"invalid field {field}: {message}")
