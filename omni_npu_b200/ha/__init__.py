"""Token recovery (high availability): survive a failed model step without dropping the
requests in flight.  See ``server`` (coordinator), ``monitor`` (worker side), ``common``."""
from .common import HAEnv  # noqa: F401
