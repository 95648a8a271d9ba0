"""Import-path compatibility: ``llm_systems.*`` resolves to the B200-native implementation."""
