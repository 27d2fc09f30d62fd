"""Search-space description shared by kernels and tuners (API of sparta/common/tuning.py:10-75)."""
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Union


@dataclass
class TunableItemCfg:
    """A ``choice`` parameter: ``_value`` lists the options (or, when ``_is_nested``, maps a
    sub-space name to a dict of ``TunableItemCfg``)."""
    _type: str
    _value: Union[Dict, List]
    _is_nested: Optional[bool] = False

    def __post_init__(self):
        assert self._type in ['choice']
        if self._is_nested:
            assert isinstance(self._value, dict)
            for sub in self._value.values():
                assert isinstance(sub, dict)
                assert all(isinstance(cfg, TunableItemCfg) for cfg in sub.values())
        else:
            assert isinstance(self._value, list)

    def includes(self, value: Any) -> bool:
        return (not self._is_nested) and value in self._value

    def to_nni_search_space(self):
        """The same space in NNI's dictionary format."""
        if not self._is_nested:
            return {'_type': self._type, '_value': self._value}
        subspaces = []
        for name, sub in self._value.items():
            entry = {'_name': name}
            entry.update({k: v.to_nni_search_space() for k, v in sub.items()})
            subspaces.append(entry)
        return {'_type': self._type, '_value': subspaces}
