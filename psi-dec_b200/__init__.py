"""B200-native paged GQA decode path of psi-dec: Python front-end of ``libpsi_cuda.so``.

The directory name carries a hyphen, so the package is loaded by path (``__graft_entry__.load_package()``) and
registered as ``psi_dec_b200``.
"""
from .binding import (  # noqa: F401
    BF16, F16, F32, CAPACITY_BUCKETED, CAPACITY_CALLER_TOKENS, CAPACITY_EXACT, KERNEL_AUTO, KERNEL_GENERIC, KERNEL_MMA, KERNEL_MMA_SYNC, KERNEL_MMA_TMA,
    PLAN_BALANCED, PLAN_REFERENCE, Context, GQA, GQAConfig, GQAPageTableLayout, KvExchange, GQAReplayShape, GQARequestPageTable,
    GQASplitKV, GQASplitKVVariant, NormRopeConfig, PageArena, PsiError, ReplayBucketPolicy, U32IDAllocator, ExecutorHibernationPlan, StateSnapshotReader, StateSnapshotWriter,
    SNAPSHOT_PAGE_ARENA, SNAPSHOT_MAIN_GQA_REQUEST_PAGE_TABLE, SNAPSHOT_MAIN_GDN_REQUEST_STATE_TABLE,
    SNAPSHOT_MTP_GQA_REQUEST_PAGE_TABLE, SNAPSHOT_DSPARK_GQA_REQUEST_PAGE_TABLE, attend_static, library, library_path, rope_parameters,
)
