"""Service layer in front of several engine instances: registry (leases, watches), load-balance policies, request router."""
from .registry import InstanceInfo, Registry  # noqa: F401
