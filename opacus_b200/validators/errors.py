"""Exception hierarchy for model validation (``opacus/validators/errors.py:17-67``)."""


class UnsupportedError(ValueError):
    """Root of everything the validator can report."""


class UnsupportedModuleError(UnsupportedError):
    """A module cannot be trained privately as it is."""


class UnsupportableModuleError(UnsupportedModuleError):
    """...and never will be (e.g. it mixes samples by construction)."""


class NotYetSupportedModuleError(UnsupportedModuleError):
    """...but support is planned."""


class ShouldReplaceModuleError(UnsupportedModuleError):
    """...but an equivalent replacement exists (see ``ModuleValidator.fix``)."""


class IllegalModuleConfigurationError(UnsupportedModuleError):
    """The module type is fine, its configuration is not."""
