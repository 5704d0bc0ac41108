// Mutation fuzzing of the JSON and TOML parsers and of the configuration loader, meant
// to run under AddressSanitizer (`make asan`). The admin endpoint parses JSON that
// arrives over TCP and the daemon parses operator-written TOML, so malformed text must
// end in an exception, never in a crash, a hang or an out-of-bounds access.
#include <stdio.h>
#include <stdlib.h>

#include <random>
#include <string>
#include <vector>

#include "../common/value.h"
#include "../daemon/config.h"

int main(int argc, char** argv) {
  const int rounds = argc > 1 ? atoi(argv[1]) : 20000;
  const std::vector<std::string> seeds_json = {
      "{\"cmd\":\"reconfig\",\"patterns\":[{\"communicator_id\":7,\"channels\":[{\"channel_id\":0,\"ring\":[1,0]}],\"ctas\":-1}]}",
      "{\"a\":[1,2.5e3,-7,true,false,null,\"x\\n\\u00e9\\\"\"],\"b\":{\"c\":{}}}",
      "{\"cmd\":\"qos_set\",\"tenants\":{\"7\":{\"weight\":2.0,\"priority\":1}},\"epoch_microsecs\":400,"
      "\"schedule\":{\"7\":{\"intervals\":[[0,100]],\"mode\":\"Deny\"}}}",
  };
  const std::vector<std::string> seeds_toml = {
      "listen_port = 5000\nmccs_daemon_prefix = \"/tmp/mccs-${USER}\"\n[control]\nprefix = \"/tmp/x\"\npath = \"c.sock\"\n"
      "[comm_default_config]\nbuffer_sizes = [4194304]\nchannel_count = 2\n[b200]\ntransport = \"auto\"\nnvls = true\n"
      "[qos.tenants.300]\nweight = 2.0\n[qos_schedule]\nepoch_microsecs = 85000\n[qos_schedule.schedule.99]\n"
      "intervals = [[0, 35000]]\nmode = \"Allow\"\n[[comm_patterns_override]]\ncommunicator_id = 138\n"
      "channels = [ { channel_id = 0, ring = [0,1,2,3], udp_sport = [[3,4,49200]], net_dev = \"mlx5_0\" } ]\n",
      "a = 1\nb = \"s\" # comment\nc = [1, 2,\n 3]\n[t]\nd = { e = 1.5, f = [true, false] }\n[[arr]]\nx = 0x10\n[[arr]]\nx = 1_000\n",
  };
  std::mt19937_64 rng(12345);
  const char alphabet[] = "{}[]\",:=.#\n\\ -0123456789eEtrufalsn'\t_x";
  long parsed = 0, rejected = 0;
  for (int i = 0; i < rounds; i++) {
    const bool toml = (i & 1) != 0;
    const auto& seeds = toml ? seeds_toml : seeds_json;
    std::string text = seeds[rng() % seeds.size()];
    const int edits = 1 + (int)(rng() % 6);
    for (int e = 0; e < edits && !text.empty(); e++) {
      const size_t pos = rng() % text.size();
      switch (rng() % 4) {
        case 0: text[pos] = alphabet[rng() % (sizeof alphabet - 1)]; break;
        case 1: text.erase(pos, 1 + rng() % 4); break;
        case 2: text.insert(pos, 1, alphabet[rng() % (sizeof alphabet - 1)]); break;
        case 3: text.insert(pos, text.substr(rng() % text.size(), rng() % 12)); break;
      }
    }
    try {
      if (toml) {
        mccs::Value v = mccs::parse_toml(text);
        try { (void)mccs::Config::from_value(v); } catch (const std::exception&) {}
        (void)v.to_json();
      } else {
        mccs::Value v = mccs::parse_json(text);
        (void)mccs::parse_json(v.to_json());   // what we print must parse again
        for (const mccs::Value& p : v["patterns"].items()) {
          try { (void)mccs::Config::parse_pattern(p); } catch (const std::exception&) {}
        }
      }
      parsed++;
    } catch (const std::exception&) {
      rejected++;
    }
  }
  // deep nesting must be refused or handled, not overflow the stack
  for (const char* open : {"[", "{\"a\":"}) {
    std::string deep;
    for (int i = 0; i < 100000; i++) deep += open;
    try { (void)mccs::parse_json(deep); } catch (const std::exception&) { rejected++; }
  }
  printf("fuzz_value: %ld parsed, %ld rejected, no crash\n", parsed, rejected);
  return 0;
}
