"""The run contract's dataclasses under the reference's package name (they live in ``research_b200.config.specs``)."""

from research_b200.config.specs import *  # noqa: F401,F403
from research_b200.config import specs as _specs
from research_b200.data.manifest import PreparedDatasetManifest as DatasetManifest  # noqa: F401
from research_b200.data.manifest import TokenShard as ShardInfo  # noqa: F401

__all__ = sorted(n for n in dir(_specs) if n[:1].isupper() and not n.startswith("_")) + ["DatasetManifest", "ShardInfo"]
