"""Import-path compatibility: ``llm_core.*`` resolves to the B200-native implementation."""
