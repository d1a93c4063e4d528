"""Plugin option tables: typed options, validators, visibility, environment and config-file overrides, finalize."""
import json

import pytest

from openvino_b200.runtime.plugin_config import ConfigOption, OptionVisibility, PluginConfig


class DemoConfig(PluginConfig):
    def declare_options(self):
        V = OptionVisibility
        self.register(ConfigOption("NUM_STREAMS", 1, "streams", lambda v: v >= -1, V.RELEASE))
        self.register(ConfigOption("PERFORMANCE_HINT", "LATENCY", "hint", lambda v: v in ("LATENCY", "THROUGHPUT"), V.RELEASE))
        self.register(ConfigOption("ENABLE_X", False, "switch", None, V.RELEASE))
        self.register(ConfigOption("QUEUE_DEPTH", 4, "internal", lambda v: 1 <= v <= 64, V.RELEASE_INTERNAL))
        self.register(ConfigOption("DUMP_DIR", "", "debug dump directory", None, V.DEBUG, str))

    def finalize_impl(self):
        if self["PERFORMANCE_HINT"] == "THROUGHPUT" and not self.is_set_by_user("NUM_STREAMS"):
            self.set_property({"NUM_STREAMS": 4})


def test_user_properties_are_typed_validated_and_frozen_by_finalize():
    c = DemoConfig()
    c.set_user_property({"NUM_STREAMS": "3", "ENABLE_X": "YES"}, OptionVisibility.RELEASE)
    assert c["NUM_STREAMS"] == 3 and c["ENABLE_X"] is True           # visible before finalize
    with pytest.raises(ValueError):
        c.set_user_property({"NUM_STREAMS": -7})
    with pytest.raises(ValueError):
        c.set_user_property({"PERFORMANCE_HINT": "FAST"})
    with pytest.raises(KeyError):
        c.set_user_property({"NO_SUCH_OPTION": 1})
    c.finalize()
    assert c["NUM_STREAMS"] == 3 and not c.is_set_by_user("NUM_STREAMS")
    with pytest.raises(RuntimeError):
        c.set_user_property({"NUM_STREAMS": 2})


def test_hint_derives_dependent_option_unless_the_user_set_it():
    a = DemoConfig()
    a.set_user_property({"PERFORMANCE_HINT": "THROUGHPUT"})
    assert a.finalize()["NUM_STREAMS"] == 4
    b = DemoConfig()
    b.set_user_property({"PERFORMANCE_HINT": "THROUGHPUT", "NUM_STREAMS": 1})
    assert b.finalize()["NUM_STREAMS"] == 1


def test_visibility_limits_what_the_public_interface_may_touch(monkeypatch):
    c = DemoConfig()
    with pytest.raises(PermissionError):
        c.set_user_property({"QUEUE_DEPTH": 8}, OptionVisibility.RELEASE)
    c.set_user_property({"QUEUE_DEPTH": 8}, OptionVisibility.RELEASE | OptionVisibility.RELEASE_INTERNAL)
    assert c["QUEUE_DEPTH"] == 8
    with pytest.raises(KeyError):                      # debug options do not exist without debug capabilities
        c.set_user_property({"DUMP_DIR": "/tmp/x"})
    monkeypatch.setenv("OVB_DEBUG_CAPS", "1")
    d = DemoConfig()
    d.set_user_property({"DUMP_DIR": "/tmp/x"})
    assert d["DUMP_DIR"] == "/tmp/x" and "DUMP_DIR" not in d.supported(OptionVisibility.RELEASE)


def test_environment_and_config_file_override(monkeypatch, tmp_path):
    path = tmp_path / "cfg.json"
    path.write_text(json.dumps({"DEMO.1": {"QUEUE_DEPTH": "16", "UNKNOWN": "1"}, "OTHER": {"QUEUE_DEPTH": "2"}}))
    monkeypatch.setenv("OV_DEBUG_CONFIG", str(path))
    monkeypatch.setenv("OV_NUM_STREAMS", "7")
    monkeypatch.setenv("OV_DUMP_DIR", "/tmp/ignored")      # debug option without debug capabilities: ignored
    c = DemoConfig()
    c.set_user_property({"NUM_STREAMS": 2})
    c.finalize(device_name="DEMO")
    assert c["QUEUE_DEPTH"] == 16 and c["NUM_STREAMS"] == 7 and c._options["DUMP_DIR"].value == ""
    monkeypatch.setenv("OV_QUEUE_DEPTH", "1000")           # the validator also guards the environment route
    with pytest.raises(ValueError):
        DemoConfig().finalize(device_name="DEMO")


def test_rt_info_applies_unless_set_by_user_and_help_lists_options():
    c = DemoConfig()
    c.apply_rt_info_property("NUM_STREAMS", {"NUM_STREAMS": "5"})
    assert c["NUM_STREAMS"] == 5
    d = DemoConfig()
    d.set_user_property({"NUM_STREAMS": 2})
    d.apply_rt_info_property("NUM_STREAMS", {"NUM_STREAMS": "5"})
    assert d["NUM_STREAMS"] == 2
    text = d.help()
    assert "QUEUE_DEPTH" in text and "RELEASE_INTERNAL" in text and "NUM_STREAMS: 2" in d.to_string()


def test_cuda_option_table():
    from openvino_b200 import properties as props
    torch = pytest.importorskip("torch")
    from openvino_b200.runtime.cuda_plugin import CudaConfig
    c = CudaConfig()
    c.set_user_property({props.hint.performance_mode: "THROUGHPUT", props.cuda.serving_program: "YES"}, OptionVisibility.RELEASE)
    c.finalize()
    assert c[props.num_streams] == 2 and c[props.cuda.serving_program] is True
    with pytest.raises(ValueError):
        CudaConfig().set_user_property({props.hint.inference_precision: "int3"})
    with pytest.raises(PermissionError):
        CudaConfig().set_user_property({"CUDA_PDL": False}, OptionVisibility.RELEASE)
