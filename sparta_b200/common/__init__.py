from sparta_b200.common.tuning import TunableItemCfg
