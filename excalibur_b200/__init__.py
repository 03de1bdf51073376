"""B200-native (sm_100a) CNN forward hot path behind the Excalibur operation interface."""
