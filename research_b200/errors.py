"""Exception hierarchy (reference: src/jaxtitan/errors.py:4-12)."""


class JaxtitanError(Exception):
    """Base class: the CLI turns it into ``error: ...`` on stderr and exit code 2."""


class ConfigError(JaxtitanError):
    """A TOML config is missing, malformed or inconsistent."""


class ContractError(JaxtitanError):
    """A runtime contract (data, checkpoint, kernel, state) was violated."""


class KernelError(ContractError):
    """A native kernel launcher refused its arguments or a device-side bounded wait ran out."""
