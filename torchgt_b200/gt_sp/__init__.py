"""Host-side mirror of the reference's ``gt_sp`` package for the sparse-attention path: sequence-parallel
state (``initialize``), edge-index and global-token helpers (``utils``) and the Ulysses layers
(``layer``, ``gt_layer``)."""
