from .connector import ConnectorMetadata, P2PKVConnector, ReqMeta, create_connector  # noqa: F401
from .manager import KVExport, KVLinkManager, make_cluster_id, parse_cluster_id  # noqa: F401
