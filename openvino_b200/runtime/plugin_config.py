"""Option tables of device plugins: typed options with defaults, validators and visibility, filled from the public
property interface, from environment variables and from a JSON configuration file, then frozen by ``finalize``.

Role of ov::PluginConfig (src/inference/dev_api/openvino/runtime/plugin_config.hpp:16-417,
src/inference/src/dev/plugin_config.cpp): a plugin declares its options once; ``set_user_property`` records what the
caller asked for (checked against the visibility that route may touch and against the option's validator);
``finalize`` copies the user's values in, lets the plugin derive dependent options (``finalize_impl``, for instance
streams from the performance hint), applies ``OV_<NAME>`` environment overrides, and freezes the result. A
configuration file (``{"CUDA": {"OPTION": "value"}}``) named by ``OV_DEBUG_CONFIG`` or passed explicitly feeds the
same options. Debug-only options are accepted when ``OVB_DEBUG_CAPS=1`` (the reference compiles them in with
ENABLE_DEBUG_CAPS).
"""
from __future__ import annotations

import enum
import json
import os
from typing import Any, Callable, Dict, Optional


class OptionVisibility(enum.IntFlag):
    RELEASE = 1            # public interface, environment and config file
    RELEASE_INTERNAL = 2   # environment and config file only
    DEBUG = 4              # debug builds only, environment and config file
    DEBUG_GLOBAL = 8       # process-wide debug option, environment only
    ANY = 0xFF


def _parse_bool(v) -> bool:
    if isinstance(v, bool):
        return v
    s = str(v).strip().upper()
    if s in ("1", "YES", "TRUE", "ON"):
        return True
    if s in ("0", "NO", "FALSE", "OFF"):
        return False
    raise ValueError("not a boolean: %r" % (v,))


_CONVERTERS: Dict[type, Callable[[Any], Any]] = {bool: _parse_bool, int: lambda v: int(str(v), 0) if isinstance(v, str) else int(v),
                                                  float: float, str: str}


class ConfigOption:
    """One option: name, default, type (taken from the default), description, validator, visibility."""

    def __init__(self, name: str, default, description: str = "", validator: Optional[Callable[[Any], bool]] = None,
                 visibility: OptionVisibility = OptionVisibility.RELEASE, type_: Optional[type] = None):
        self.name, self.default, self.description, self.validator, self.visibility = name, default, description, validator, visibility
        self.type = type_ or type(default)
        self.value = default

    def convert(self, v):
        conv = _CONVERTERS.get(self.type)
        try:
            out = conv(v) if conv else v
        except (TypeError, ValueError) as e:
            raise ValueError("option %s: cannot convert %r to %s (%s)" % (self.name, v, self.type.__name__, e))
        if self.validator is not None and not self.validator(out):
            raise ValueError("option %s: invalid value %r" % (self.name, v))
        return out

    def is_valid_value(self, v) -> bool:
        try:
            self.convert(v)
            return True
        except ValueError:
            return False


class PluginConfig:
    env_prefix = "OV_"

    def __init__(self):
        self._options: Dict[str, ConfigOption] = {}
        self._user: Dict[str, Any] = {}
        self._finalized = False
        self.declare_options()

    # ---- declaration (sub-classes override declare_options and call register)
    def declare_options(self) -> None:
        pass

    def register(self, option: ConfigOption) -> ConfigOption:
        self._options[option.name] = option
        return option

    def _debug_caps(self) -> bool:
        return os.environ.get("OVB_DEBUG_CAPS", "") == "1"

    def _option(self, name: str) -> ConfigOption:
        opt = self._options.get(name)
        if opt is None or (opt.visibility in (OptionVisibility.DEBUG, OptionVisibility.DEBUG_GLOBAL) and not self._debug_caps()):
            raise KeyError("Option not found: %s" % name)
        return opt

    # ---- access
    def set_user_property(self, properties: Dict[str, Any], allowed_visibility: OptionVisibility = OptionVisibility.ANY, strict: bool = True) -> None:
        """Record what a caller asked for. ``allowed_visibility`` is what the route the request came through may touch: the
        public ``set_property`` / ``compile_model`` interface passes RELEASE."""
        if self._finalized:
            raise RuntimeError("the configuration is finalized")
        for name, value in properties.items():
            try:
                opt = self._option(name)
            except KeyError:
                if strict:
                    raise
                continue
            if not (opt.visibility & allowed_visibility):
                raise PermissionError("option %s (%s) cannot be set through this interface" % (name, opt.visibility.name))
            self._user[name] = opt.convert(value)

    def set_property(self, properties: Dict[str, Any]) -> None:
        """Internal assignment (plugin code, environment, config file): validated, no visibility check."""
        for name, value in properties.items():
            opt = self._option(name)
            opt.value = opt.convert(value)

    def get_property(self, name: str, allowed_visibility: OptionVisibility = OptionVisibility.ANY):
        opt = self._option(name)
        if not (opt.visibility & allowed_visibility):
            raise PermissionError("option %s (%s) is not readable through this interface" % (name, opt.visibility.name))
        if not self._finalized and name in self._user:
            return self._user[name]
        return opt.value

    def __getitem__(self, name: str):
        return self.get_property(name)

    def is_set_by_user(self, name: str) -> bool:
        return name in self._user

    def supported(self, visibility: OptionVisibility = OptionVisibility.RELEASE):
        return [n for n, o in self._options.items() if o.visibility & visibility]

    # ---- sources
    def read_env(self) -> Dict[str, str]:
        out = {}
        for name, opt in self._options.items():
            if opt.visibility in (OptionVisibility.DEBUG, OptionVisibility.DEBUG_GLOBAL) and not self._debug_caps():
                continue
            v = os.environ.get(self.env_prefix + name, "")
            if v != "":
                out[name] = v
        return out

    def read_config_file(self, path: str, device_name: str) -> Dict[str, str]:
        """``{"<DEVICE>[.id]": {"OPTION": "value", ...}, ...}``; sections of other devices and unreadable files are ignored."""
        if not path:
            return {}
        try:
            with open(path) as f:
                data = json.load(f)
        except (OSError, ValueError):
            return {}
        out = {}
        want = device_name.split(".")[0]
        for dev, section in data.items() if isinstance(data, dict) else []:
            if dev.split(".")[0] != want or not isinstance(section, dict):
                continue
            for k, v in section.items():
                out[k] = v if isinstance(v, str) else json.dumps(v)
        return out

    def _cleanup_unsupported(self, cfg: Dict[str, Any]) -> Dict[str, Any]:
        return {k: v for k, v in cfg.items() if k in self._options and self._options[k].visibility != OptionVisibility.DEBUG_GLOBAL
                and (self._options[k].visibility != OptionVisibility.DEBUG or self._debug_caps())}

    def apply_env_options(self) -> None:
        self.set_property(self._cleanup_unsupported(self.read_env()))

    def apply_config_options(self, device_name: str, path: Optional[str] = None) -> None:
        path = path if path is not None else os.environ.get("OV_DEBUG_CONFIG", "")
        self.set_property(self._cleanup_unsupported(self.read_config_file(path, device_name)))

    # ---- freezing
    def apply_model_specific_options(self, model) -> None:
        pass

    def finalize_impl(self) -> None:
        pass

    def finalize(self, model=None, device_name: str = "") -> "PluginConfig":
        if self._finalized:
            return self
        if model is not None:
            self.apply_model_specific_options(model)
        for name, value in self._user.items():
            self._options[name].value = value
        self.finalize_impl()
        if device_name:
            self.apply_config_options(device_name)
        self.apply_env_options()
        self._user.clear()
        self._finalized = True
        return self

    def apply_rt_info_property(self, name: str, rt_info: Dict[str, Any]) -> None:
        """A value stored in the model's rt_info applies unless the user set the option explicitly."""
        if not self.is_set_by_user(name) and name in rt_info:
            self.set_user_property({name: rt_info[name]}, OptionVisibility.RELEASE)

    def clone(self) -> "PluginConfig":
        c = type(self)()
        for n, o in self._options.items():
            c._options[n].value = o.value
        c._user = dict(self._user)
        return c

    def to_dict(self) -> Dict[str, Any]:
        return {n: (self._user[n] if (not self._finalized and n in self._user) else o.value) for n, o in self._options.items()}

    def to_string(self) -> str:
        return "\n".join("%s: %s" % (k, v) for k, v in sorted(self.to_dict().items()))

    def help(self, name: str = "") -> str:
        opts = [self._options[name]] if name else list(self._options.values())
        return "\n".join("%-36s %-16s default=%r  %s" % (o.name, o.visibility.name, o.default, o.description) for o in opts)
