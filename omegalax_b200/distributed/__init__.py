"""Import path of the reference's mesh helpers (``omegalax.distributed.mesh``): the same module
as ``omegalax_b200.parallel.mesh``, so that ``from omegalax_b200.distributed import mesh`` and
``from omegalax_b200.distributed.mesh import ensure_mesh`` keep working for code written against
the reference layout."""
import sys

from ..parallel import mesh

sys.modules[__name__ + ".mesh"] = mesh
