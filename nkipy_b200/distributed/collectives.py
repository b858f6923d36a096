"""Collective operations usable inside kernels
(nkipy/src/nkipy/distributed/collectives.py:4-11 in the reference).

    all_gather(data, all_gather_dim, replica_groups)
    all_reduce(data, replica_groups, reduce_op=np.add)
    reduce_scatter(data, reduce_scatter_dim, replica_groups, reduce_op=np.add)
    all_to_all(data, split_dimension, concat_dimension, replica_groups)

While tracing they become IR collective nodes; called on NumPy arrays they evaluate
for a single process under the "every rank holds the same data" convention.
"""

from ..core.ops import all_gather, all_reduce, all_to_all, reduce_scatter

__all__ = ["all_gather", "all_reduce", "reduce_scatter", "all_to_all"]
