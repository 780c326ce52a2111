"""chaoscontrol_b200: a Blackwell-native (sm_100a) diagonal-SSM language-model
framework with the capabilities and public API of KenMalloy/chaoscontrol."""
__version__ = "0.1.0"
