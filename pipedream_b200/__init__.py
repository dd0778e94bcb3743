"""pipedream_b200: B200-native pipeline-parallel training step with the PipeDream runtime API.

Public modules mirror the reference's runtime package: `runtime` (StageRuntime),
`optimizer` / `sgd` / `adam` (weight stashing), `communication`
(CommunicationHandler).  The compute runs in libpipedream_b200.so (C-ABI,
sm_100a); importing the package does not load it, the first kernel call does.
"""
__version__ = "0.1.0"
