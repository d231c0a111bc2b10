"""Distribution runtime: the ('expert', 'replica') process mesh, expert all-to-all exchange,
named barrier, regex-driven parameter placement and gradient reduction."""
from vmoe_b200.parallel.mesh import (Mesh, get_auto_logical_mesh, get_mesh, init_distributed,
                                     log_logical_mesh, set_mesh, use_mesh)
from vmoe_b200.parallel.exchange import ExpertExchange, LOCAL_EXCHANGE
from vmoe_b200.parallel.multihost_utils import sync_devices
from vmoe_b200.parallel.partitioning import (PartitionSpec, parse_partition_spec,
                                             tree_axis_resources_from_regexes)
