from .engine_entry import RoleInfo, build_arm_config, init_arm_topology, run_arm_submission

__all__ = ["RoleInfo", "build_arm_config", "init_arm_topology", "run_arm_submission"]
